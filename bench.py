#!/usr/bin/env python
"""Benchmark of the FP8 block-scale DeepSeek-V3 MoE shard on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
    python bench.py --replay ROOT|synthetic      # a flashinfer-trace workload set, per-workload table
    python bench.py --profile-only --workload NAME   # W + K bare calls on one weight replica (profiler captures)

One step = one call of the operator on one batch of seeded synthetic tokens.
N = 1 measures the decode workload (T = 1, the configuration the headline metric
is quoted on) and carries the other single-GPU workloads as `sweep` rows; N > 1
(under torchrun) measures the 256-expert layer with expert parallelism over N GPUs
(T = 16384 tokens; dispatch and combine over NVLink peer memory, the NCCL all-to-all
transport timed beside it).  Rank 0 prints ONE JSON line.

Every measured row carries `parity` (the CUDA result against the oracle on the same
inputs) and `roofline` (achieved HBM GB/s and FP8 TFLOP/s of the dominant kernel
against the measured peaks).  `--impl reference` times the definition's CPU path on
the host cores on the same workload.

Timing: CUDA events on the launching stream around the K timed steps (W warm-up
steps before), max over ranks.  A decode step touches < 126 MB of weights, so
consecutive steps rotate through R replicas of the shard's weights (different
addresses, same values) chosen so that a replica is reused only after more
than 3x the L2 capacity has been streamed: every step reads its weights from HBM
("inputs larger than L2"), without a flush kernel leaving dirty lines behind.
"""
from __future__ import annotations

import argparse
import importlib.util
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
H = 7168

# single-GPU workloads (the benchmark specification's configs 1, 0, 2, 3 and two sizes in between)
WORKLOADS = {
    "decode_t1":     dict(T=1, token_seed=3, skew=False),    # seed 3: first seed whose token has a local expert
    "cpu_ref_t8":    dict(T=8, token_seed=0, skew=False),
    "small_t16":     dict(T=16, token_seed=0, skew=False),
    "skew_t64":      dict(T=64, token_seed=0, skew=True),
    "mid_t512":      dict(T=512, token_seed=0, skew=False),
    "prefill_t4096": dict(T=4096, token_seed=0, skew=False),
}
EP_T = 16384                  # tokens of the expert-parallel layer workload (the specification's config 4)
EP_REFERENCE_SAMPLE = 4       # tokens of it that the CPU arm pushes through all 256 experts per step

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from ncu captures of the
# same command (None where no capture of that workload exists).
NCU_TRAFFIC_BYTES = {"decode_t1": 88_247_000 + 3_136_000,        # decode_kernel
                     "skew_t64": 473_900_000 + 12_800_000,       # grouped_gemm_kernel<1,64>
                     "mid_t512": 593_900_000 + 7_900_000,        # grouped_gemm_kernel<1,64>
                     "prefill_t4096": 829_100_000 + 35_300_000}  # grouped_gemm_large_kernel<1>

W13_BYTES = 4096 * 7168 + 32 * 56 * 4          # one expert's GEMM1 weights + scales
W2_BYTES = 7168 * 2048 + 56 * 16 * 4
ROW_BYTES = 7168 + 56 * 4                      # one activation row + its scales
FLOPS1 = 2 * 7168 * 4096                       # per (token, expert) row
FLOPS2 = 2 * 2048 * 7168
L2_BYTES = 126 << 20


def measured_peaks():
    """HBM copy bandwidth and dense bf16 throughput measured on this pool's B200s.  No FP8 peak is measured:
    the FP8 denominator is twice the bf16 burst figure (the dense e4m3 rate of the tensor core is twice its
    bf16 rate), labelled as such."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, bf16, kind = 6650.0, 1590.0, "fallback"
    if os.path.exists(p):
        try:
            j = json.load(open(p))
            hbm, bf16, kind = float(j["hbm_gbs"]), float(j["bf16_tflops"]), "measured"
        except Exception:
            pass
    return {"hbm_gbs": hbm, "fp8_tflops": 2.0 * bf16, "kind": kind,
            "fp8_kind": f"2 x {kind} bf16 burst ({bf16:.1f} TFLOP/s); no FP8 peak is measured on this pool"}


def roofline(kernel, nbytes, flops, launch_us, traffic, P, **extra):
    """Both fractions of one kernel launch; `bound` is the larger one (the resource closer to its limit)."""
    gbs = nbytes / launch_us / 1e3
    tfs = flops / launch_us / 1e6
    fh, ft = gbs / P["hbm_gbs"], tfs / P["fp8_tflops"]
    hbm_bound = fh >= ft
    d = {"bound": "hbm" if hbm_bound else "tensor", "kernel": kernel,
         "achieved": gbs if hbm_bound else tfs, "peak": P["hbm_gbs"] if hbm_bound else P["fp8_tflops"],
         "unit": "GB/s" if hbm_bound else "TFLOP/s", "frac": fh if hbm_bound else ft,
         "peak_kind": P["kind"] if hbm_bound else P["fp8_kind"], "traffic": traffic,
         "algorithmic_bytes_per_launch": nbytes, "algorithmic_flops_per_launch": flops, "launch_us": launch_us,
         "hbm": {"achieved_gbs": gbs, "peak_gbs": P["hbm_gbs"], "frac": fh, "peak_kind": P["kind"]},
         "fp8": {"achieved_tflops": tfs, "peak_tflops": P["fp8_tflops"], "frac": ft, "peak_kind": P["fp8_kind"]}}
    d.update(extra)
    return d


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples during the timed region."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int, enabled: bool = True):
        self.index, self.lines, self.proc, self.first, self.enabled = index, [], None, 0, enabled

    def __enter__(self):
        if not self.enabled:      # multi-rank runs: one poller (rank 0's) is enough, eight perturb the launches
            return self
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            # nvidia-smi needs a few hundred ms before its first line (longer on an 8-GPU box); a short timed
            # region would otherwise end without a sample.  Wait for the first line, then count from there.
            t0 = time.time()
            while not self.lines and time.time() - t0 < 5.0:
                time.sleep(0.005)
            self.first = len(self.lines)
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.03)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        lines = self.lines[self.first:] or self.lines       # samples taken after the region began (else: all)
        for ln in lines:
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


def algorithmic_bytes(T, n_active, n_tokens_with_local):
    """Bytes the operator must move: active experts' weights and scales, the
    activation rows it reads once, the routing logits and the bf16 output."""
    return n_active * (W13_BYTES + W2_BYTES) + n_tokens_with_local * ROW_BYTES + T * 1024 + T * 7168 * 2


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


def n_replicas(touched_bytes):
    n = 1
    while n < 8 and touched_bytes * (n - 1) < 3 * L2_BYTES:
        n += 1
    return n


def weight_replicas(W, touched_bytes):
    """Enough copies of the shard's weights that a copy is reused after > 3 x L2 of other traffic."""
    reps = [W]
    for _ in range(n_replicas(touched_bytes) - 1):
        reps.append(type(W)(W.gemm1_weights.clone(), W.gemm1_weights_scale.clone(), W.gemm2_weights.clone(),
                            W.gemm2_weights_scale.clone()))
    return reps


def wtuple(w):
    return (w.gemm1_weights, w.gemm1_weights_scale, w.gemm2_weights, w.gemm2_weights_scale)


def workload_config(name, n_sel, n_active):
    """The `config` block of a single-GPU line; both arms print exactly this."""
    wl = WORKLOADS[name]
    R = n_replicas(max(1, n_active) * (W13_BYTES + W2_BYTES))
    return {"workload": name, "T": wl["T"], "token_seed": wl["token_seed"], "weight_seed": 0,
            "routing_skew": wl["skew"], "local_expert_offset": 0, "n_sel": int(n_sel),
            "active_experts": int(n_active),
            "l2": f"{R} weight replicas rotated: {R * n_active * (W13_BYTES + W2_BYTES) >> 20} MiB "
                  "streamed per cycle > 3 x 126 MB L2"}


def ep_config(world):
    """The `config` block of an expert-parallel line; both arms print exactly this."""
    return {"workload": f"ep_layer_t{EP_T}", "T": EP_T, "tokens_per_rank": EP_T // world, "experts": 256,
            "shards_per_rank": 8 // world, "token_seed": 0, "weight_seeds": "1000 + shard",
            "l2": "per-rank weights (>= 1.4 GB) exceed L2"}


def load_oracle():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import moe_oracle
    return moe_oracle


def load_definition():
    """The reference's own PyTorch definition, when a copy was placed under oracle/_ref/ (oracle/make_ref.py)."""
    f = os.path.join(ROOT, "oracle", "_ref", "moe_definition.py")
    if not os.path.exists(f):
        return None
    spec = importlib.util.spec_from_file_location("moe_definition", f)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def oracle_check(oracle, tok, W, out, T):
    """Parity of `out` against the oracle on the same inputs: on the host for small batches, on the GPU in
    fp32 (TF32 off) for large ones.  Returns (metrics, oracle result)."""
    if T <= 64:
        cpu_tok = [t.cpu() for t in (tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale)]
        wt = wtuple(W)
        cache = {}

        def ew(le):
            if le not in cache:
                cache[le] = tuple(x[le].cpu() for x in wt)
            return cache[le]
        ref = oracle.run(*cpu_tok, ew, 0, RSF)
        where = "cpu"
    else:
        torch.backends.cuda.matmul.allow_tf32 = False
        ref = oracle.run_full(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale,
                              *wtuple(W), 0, RSF)
        where = "gpu_fp32"
    m = oracle.output_metrics(out, ref.output, ref.output_f32)
    assert m["cosine"] >= 0.9999 and m["match_ratio"] >= 0.999, m
    rep = oracle.parity_report(m)
    rep["oracle_on"] = where
    return rep, ref


def gemm_rooflines(sched, stage_us, P, large=False, fast_combine=False):
    """Roofline blocks of the two grouped GEMM launches of the general path from the stage events."""
    k1 = "grouped_gemm_large_kernel<1> (GEMM1 + SwiGLU + e4m3 plane split)" if large else \
        f"grouped_gemm_kernel<1,{sched.n_tile}>"
    k2 = ("grouped_gemm_large_kernel<2,combine> (GEMM2 + routing weight + fp32 combine + bf16 cast)" if fast_combine
          else "grouped_gemm_large_kernel<2>") if large else f"grouped_gemm_kernel<2,{sched.n_tile2}>"
    g1 = roofline(k1, sched.n_active * W13_BYTES + sched.n_sel * ROW_BYTES, sched.n_sel * FLOPS1, stage_us["gemm1"], None, P)
    g2 = roofline(k2, sched.n_active * W2_BYTES, sched.n_sel * FLOPS2, stage_us["gemm2"], None, P)
    return g1, g2


def profile_stages(loader, step, n):
    loader.set_profiling(True)
    acc = {}
    for i in range(n + 3):
        step(i)
        st = loader.stage_times_ms()
        if i >= 3:
            for k, v in st.items():
                acc[k] = acc.get(k, 0.0) + v
    loader.set_profiling(False)
    return {k: v / n * 1e3 for k, v in acc.items()}


def measure_workload(pkg, oracle, W, name, steps, warmup, P, nprof=10, options=0):
    """One single-GPU workload: tokens/s with resident inputs, per-stage times, roofline, parity.
    `options`: operator options (MOE_B200_OPT_*) in force for this measurement only."""
    gen, op, loader = pkg.gen, pkg.op, pkg.loader
    loader.set_options(options)
    try:
        return _measure_workload(pkg, oracle, W, name, steps, warmup, P, nprof, options)
    finally:
        loader.set_options(0)


def _measure_workload(pkg, oracle, W, name, steps, warmup, P, nprof, options):
    gen, op, loader = pkg.gen, pkg.op, pkg.loader
    dev = W.gemm1_weights.device
    wl = WORKLOADS[name]
    T = wl["T"]
    tok = gen.make_tokens(T, wl["token_seed"], dev, wl["skew"])
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    # one untimed call tells how many experts the batch touches, which sizes the replica ring
    op.run(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale, *wtuple(W), 0, RSF, out)
    sched = op.read_schedule(T)
    reps = weight_replicas(W, max(1, sched.n_active) * (W13_BYTES + W2_BYTES))
    R = len(reps)

    def step(i=0):
        op.run(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale,
               *wtuple(reps[i % R]), 0, RSF, out)

    launches0 = loader.launch_count()
    with ClockSampler(0) as clocks:
        ms_step = time_steps(step, steps, warmup)
    launches = (loader.launch_count() - launches0) * steps // (steps + warmup)
    assert op.kernel_status() == 0
    sched = op.read_schedule(T)
    stage_us = profile_stages(loader, step, nprof)
    _, _, mask = op.route(tok.routing_logits, tok.routing_bias, 0, RSF)
    n_local_tokens = int((mask != 0).sum())
    op_bytes = algorithmic_bytes(T, sched.n_active, n_local_tokens)
    op_flops = sched.n_sel * (FLOPS1 + FLOPS2)
    us = ms_step * 1e3
    whole = roofline("whole operator (all launches of one step)", op_bytes, op_flops, us, None, P)
    if T <= 16:
        # one launch per step: the kernel's average launch duration is the timed region / K
        dom = roofline("decode_kernel: routing + GEMM1 + SwiGLU + GEMM2 + combine in one launch", op_bytes, op_flops,
                       us, NCU_TRAFFIC_BYTES.get(name), P)
        kernels = {}
    else:
        g1, g2 = gemm_rooflines(sched, stage_us, P, large=T > 1024 and not (options & loader.OPT_UNFUSED),
                                fast_combine=bool(options & loader.OPT_FAST_COMBINE))
        dom = g1 if stage_us["gemm1"] >= stage_us["gemm2"] else g2
        dom["traffic"] = NCU_TRAFFIC_BYTES.get(name) if dom is g1 else None
        kernels = {"gemm1": g1, "gemm2": g2}
    step(0)       # leave `out` holding replica 0's result for the check
    torch.cuda.synchronize()
    parity, ref = oracle_check(oracle, tok, W, out, T)
    row = {"workload": name, "options": {"fast_combine": bool(options & loader.OPT_FAST_COMBINE),
                                         "unfused": bool(options & loader.OPT_UNFUSED)},
           "T": T, "n_sel": sched.n_sel, "active_experts": sched.n_active, "replicas": R,
           "us_per_step": us, "tokens_per_s": T / us * 1e6, "gpu_launches_per_step": launches // max(1, steps),
           "split_k": [sched.split1, sched.split2], "token_tile": [sched.n_tile, sched.n_tile2],
           "stage_us": stage_us, "roofline": dom, "whole_op": whole, "kernels": kernels, "parity": parity}
    return row, dict(tok=tok, out=out, reps=reps, step=step, sched=sched, clocks=clocks, launches=launches, ref=ref)


def cpu_baseline(pkg, oracle, tok, W, sched, T):
    """The definition on the host cores, on a bounded sample of the same workload (about 10-30 s)."""
    cpu_tok = [t.cpu() for t in (tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale)]
    definition = load_definition()
    threads = torch.get_num_threads()
    if definition is not None:
        cpu_w = [x.cpu() for x in wtuple(W)]
        t0 = time.time()
        calls = 0
        while True:
            ref_out = definition.run(*cpu_tok, *cpu_w, 0, RSF)
            calls += 1
            if time.time() - t0 > 15.0 or calls >= 3:
                break
        dt = time.time() - t0
        port = oracle.run_full(*cpu_tok, *cpu_w, 0, RSF)
        same = bool(torch.equal(ref_out.view(torch.int16), port.output.view(torch.int16)))
        return {"value": calls * T / dt, "unit": UNIT, "cores": threads, "kind": "reference",
                "sample": f"{calls} call(s) of the unmodified definition (all 32 experts dequantised) on the same "
                          f"T={T} batch ({dt:.1f} s)",
                "oracle_port_bit_identical_to_definition": same}
    active = [le for le in range(32) if sched.counts[le] > 0]
    cpu_w = {le: tuple(x[le].cpu() for x in wtuple(W)) for le in active}
    t0 = time.time()
    calls = 0
    while True:
        oracle.run(*cpu_tok, lambda le: cpu_w[le], 0, RSF)
        calls += 1
        if time.time() - t0 > 10.0 or calls >= 50:
            break
    dt = time.time() - t0
    return {"value": calls * T / dt, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{calls} calls of the oracle port on the same T={T} batch ({dt:.1f} s); "
                      "only the experts the batch uses are dequantised"}


def oracle_vs_oracle(pkg, oracle, dev):
    """Two faithful fp32 evaluations of the definition against each other (GPU cuBLAS fp32 vs CPU), T = 64
    skewed: what the literal max-abs bar reads for an implementation that is not the CUDA path at all."""
    gen = pkg.gen
    tok = gen.make_tokens(64, 0, dev, True)
    Wg = gen.make_shard_weights(0, dev, experts=range(16))
    torch.backends.cuda.matmul.allow_tf32 = False
    g = oracle.run_full(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale, *wtuple(Wg),
                        0, RSF)
    cpu = lambda t: t.cpu()
    c = oracle.run(cpu(tok.routing_logits), cpu(tok.routing_bias), cpu(tok.hidden_states), cpu(tok.hidden_states_scale),
                   lambda le: tuple(cpu(x[le]) for x in wtuple(Wg)), 0, RSF)
    rep = oracle.parity_report(oracle.output_metrics(g.output, c.output, c.output_f32))
    rep["what"] = "oracle on GPU (fp32, TF32 off) vs oracle on CPU, skew_t64 inputs; no CUDA kernel of this repo involved"
    return rep


def profile_only(args):
    """W + K back-to-back steps of one single-GPU workload on ONE weight replica, nothing else."""
    pkg = load_package()
    gen, op = pkg.gen, pkg.op
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    name = args.workload or "decode_t1"
    wl = WORKLOADS[name]
    T = wl["T"]
    tok = gen.make_tokens(T, wl["token_seed"], dev, wl["skew"])
    _, _, mask = op.route(tok.routing_logits, tok.routing_bias, 0, RSF)
    used = 0
    for m in mask.cpu().tolist():
        used |= m & 0xFFFFFFFF
    W = gen.make_shard_weights(0, dev, experts=[le for le in range(32) if (used >> le) & 1])
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
    ms = time_steps(lambda i: op.run(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale,
                                     *wtuple(W), 0, RSF, out), args.steps, args.warmup)
    assert op.kernel_status() == 0
    print(json.dumps({"workload": name, "T": T, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                      "note": "profile-only run: one weight replica, no L2 rotation; not a benchmark value"}))


def bench_single(args):
    pkg = load_package()
    gen, op, loader = pkg.gen, pkg.op, pkg.loader
    oracle = load_oracle()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    P = measured_peaks()
    name = args.workload or "decode_t1"
    T = WORKLOADS[name]["T"]
    W = gen.make_shard_weights(0, dev)
    row, ctx = measure_workload(pkg, oracle, W, name, args.steps, args.warmup, P, nprof=max(10, min(args.steps, 100)))
    tok, reps, sched = ctx["tok"], ctx["reps"], ctx["sched"]
    R = len(reps)

    # ---- host buffers through the host entry point: `e2e`
    pin = lambda t: t.cpu().pin_memory()
    h = [pin(tok.routing_logits), pin(tok.routing_bias), pin(tok.hidden_states), pin(tok.hidden_states_scale)]
    out_h = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()

    def step_host(i=0):
        op.run_host(*h, *wtuple(reps[i % R]), 0, RSF, out_h)

    ms_host = time_steps(step_host, args.steps, args.warmup)
    h2d = sum(t.numel() * t.element_size() for t in h)
    d2h = out_h.numel() * out_h.element_size()

    line = {
        "metric": METRIC, "value": row["tokens_per_s"], "unit": UNIT, "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": row["us_per_step"] * 1e-3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": workload_config(name, sched.n_sel, sched.n_active),
        "run_info": {"split_k": row["split_k"], "token_tile": row["token_tile"], "replicas": R},
        "e2e": {"value": T / (ms_host * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_host,
                "note": "token tensors from pinned host memory, bf16 output read back; weights stay resident"},
        "gpu_launches": int(ctx["launches"]),
        "clocks": ctx["clocks"].summary(),
        "roofline": row["roofline"], "whole_op": row["whole_op"], "kernels": row["kernels"],
        "stage_us": row["stage_us"],
        "cpu_baseline": cpu_baseline(pkg, oracle, tok, W, sched, T),
        "parity": row["parity"],
    }
    if args.sweep:
        rows = []
        for n in WORKLOADS:
            if n != name:
                r, c = measure_workload(pkg, oracle, W, n, 30, 5, P)
                rows.append(r)
                del c
        # the large-batch path's two other modes on the prefill workload: combine fused into GEMM2's epilogue
        # (not bit-reproducible), and the multi-kernel path without any epilogue fusion (A/B)
        line["sweep_modes"] = [measure_workload(pkg, oracle, W, "prefill_t4096", 30, 5, P, options=o)[0]
                               for o in (loader.OPT_FAST_COMBINE, loader.OPT_UNFUSED)]
        line["sweep"] = rows
        line["oracle_vs_oracle"] = oracle_vs_oracle(pkg, oracle, dev)
        del W, reps, ctx
        torch.cuda.empty_cache()
        line["scale_anchor"] = ep_single_gpu(pkg, oracle, dev, min(args.steps, 20), min(max(args.warmup, 3), 5), P)
        torch.cuda.empty_cache()
        # the reference's CUDA solution on the same workloads, same box, same protocol (30 steps after 5)
        ref_rows = reference_cuda_rows()
        line["reference_cuda"] = ref_rows
        ours = {name: row["us_per_step"]}
        ours.update({r["workload"]: r["us_per_step"] for r in rows})
        if "unavailable" not in ref_rows:
            line["speedup_vs_reference_cuda"] = {n: ref_rows[n]["us_per_step"] / ours[n] for n in ours if n in ref_rows}
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# The 256-expert layer (the specification's config 4): one GPU (scale anchor) and N > 1 under torchrun
# ---------------------------------------------------------------------------------------------
def layer_parity(oracle, ep, tok_all, weights, shards, world, out, sl):
    """This rank's rows of the layer output against the layer reference: every rank runs the oracle on the GPU
    (fp32, TF32 off) for the shards it owns over ALL tokens, the bf16 shard outputs are summed over ranks in
    float64 (exact for eight bf16 terms), and the result is compared on the rank's own token slice."""
    import torch.distributed as dist
    torch.backends.cuda.matmul.allow_tf32 = False
    dev = out.device
    part = torch.zeros(tok_all.routing_logits.shape[0], H, dtype=torch.float64, device=dev)
    for w, s in zip(weights, shards):
        r = oracle.run_full(tok_all.routing_logits, tok_all.routing_bias, tok_all.hidden_states,
                            tok_all.hidden_states_scale, *wtuple(w), 32 * s, RSF)
        part += r.output.to(torch.float64)
        del r
    if world > 1:
        dist.all_reduce(part)
    ref = part[sl].to(torch.float32)
    del part
    m = oracle.output_metrics(out, ref.to(torch.bfloat16), ref)
    return oracle.parity_report(m)


def merge_parity(reports):
    """Worst case over ranks of the per-rank reports (counts are summed)."""
    out = {}
    for k in reports[0]:
        vals = [r[k] for r in reports]
        if k in ("cosine", "match_ratio"):
            out[k] = min(vals)
        elif k.startswith("n"):
            out[k] = int(sum(vals))
        else:
            out[k] = max(vals)
    return out


def check_layer_parity(rep):
    """Hard bars of the benchmark run (the tighter element-wise bars are the GPU tests')."""
    assert rep["cosine"] >= 0.9999 and rep["match_ratio"] >= 0.999, rep


def ep_single_gpu(pkg, oracle, dev, steps, warmup, P):
    """The 256-expert layer of the multi-GPU workload (T = 16384) on ONE GPU: eight shard calls per layer
    call, no communication.  The N = 1 point of the expert-parallel scaling curve, timed like the N > 1 lines."""
    gen, ep, op, loader = pkg.gen, pkg.ep, pkg.op, pkg.loader
    weights = [gen.make_shard_weights(1000 + s, dev) for s in range(8)]
    tok = gen.make_tokens(EP_T, 0, dev)
    layer = ep.ExpertParallelMoE(weights, 0, 1)

    def step(i=0):
        return layer.forward(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale, RSF)
    ms = time_steps(step, steps, warmup)
    out = step()
    assert op.kernel_status(device=dev) == 0
    rows = int(sum(layer.last_plan.recv_counts))
    parity = layer_parity(oracle, ep, tok, weights, list(range(8)), 1, out, slice(0, EP_T))
    check_layer_parity(parity)
    return {"workload": f"ep_layer_t{EP_T}", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms,
            "tokens_per_s": EP_T / (ms * 1e-3), "records": rows, "parity": parity,
            "per_gpu": roofline("whole layer call on this GPU (8 shard calls)", 8 * 32 * (W13_BYTES + W2_BYTES),
                                rows * (FLOPS1 + FLOPS2), ms * 1e3, None, P)}


def bench_ep(args):
    import torch.distributed as dist
    pkg = load_package()
    gen, loader, op, ep = pkg.gen, pkg.loader, pkg.op, pkg.ep
    oracle = load_oracle()
    P = measured_peaks()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl", device_id=dev)
    T = EP_T // world
    shards = ep.shards_of_rank(rank, world)
    weights = [gen.make_shard_weights(1000 + s, dev) for s in shards]
    tok_all = gen.make_tokens(EP_T, 0, dev)
    sl = slice(rank * T, (rank + 1) * T)
    logits = tok_all.routing_logits[sl].contiguous()
    hidden = tok_all.hidden_states[sl].contiguous()
    hscale = tok_all.hidden_states_scale[:, sl].contiguous()
    bias = tok_all.routing_bias
    transports = [os.environ.get("MOE_B200_EP_TRANSPORT", "p2p")]
    if transports[0] == "p2p":
        transports.append("nccl")          # also timed, reported beside the headline

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        t = torch.tensor([float(x)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    results, outs = {}, {}
    clocks = None
    for tr in transports:
        layer = ep.ExpertParallelMoE(weights, rank, world, transport=tr)

        def step():
            return layer.forward(logits, bias, hidden, hscale, RSF)

        for _ in range(args.warmup):
            step()
        sync()
        l0 = loader.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank, enabled=(rank == 0 and clocks is None)) as cs:
            sync()      # rank 0 waited for its sampler's first line: the ranks start the timed steps together
            e0.record()
            for _ in range(args.steps):
                out = step()
            e1.record()
            sync()
        if clocks is None:
            clocks = cs.summary()
        n_rows = torch.tensor([float(sum(layer.last_plan.recv_counts))], device=dev)
        rows_max = n_rows.clone()
        if world > 1:
            dist.all_reduce(rows_max, op=dist.ReduceOp.MAX)
            dist.all_reduce(n_rows, op=dist.ReduceOp.SUM)
        results[tr] = dict(ms_step=max_over_ranks(e0.elapsed_time(e1)) / args.steps,
                           launches=loader.launch_count() - l0, rows=float(n_rows), rows_max=float(rows_max),
                           digest=gen.digest(out))
        outs[tr] = out
        if tr == transports[0]:
            # one profiled call: stage events of this rank's LAST shard call (the dominant kernel's roofline)
            loader.set_profiling(True)
            step()
            stage_ms = loader.stage_times_ms()
            loader.set_profiling(False)
            shard_rows = layer.last_shard_rows[-1]
            shard_sched = op.read_schedule(shard_rows) if shard_rows > 0 else None
        del layer
    assert op.kernel_status(device=dev) == 0
    if len(results) == 2:
        assert results["p2p"]["digest"] == results["nccl"]["digest"], "transports disagree"

    # ---- the same layer from bf16 activations: the dispatch kernel quantises every token on its way out.  The bf16
    # rows are the ones the generator quantised into `hidden`, so the output must have the same bits.
    bf16_dispatch = None
    if transports[0] == "p2p":
        x_all = gen.normal(0, gen._S_HIDDEN, 0, EP_T * H, dev).view(EP_T, H).to(torch.bfloat16)
        x = x_all[sl].contiguous()
        del x_all
        layer = ep.ExpertParallelMoE(weights, rank, world, transport="p2p")
        for _ in range(args.warmup):
            out_b = layer.forward_bf16(logits, bias, x, RSF)
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            out_b = layer.forward_bf16(logits, bias, x, RSF)
        e1.record()
        sync()
        assert gen.digest(out_b) == results["p2p"]["digest"], "bf16 dispatch changed the result"
        bf16_dispatch = {"ms_per_step": max_over_ranks(e0.elapsed_time(e1)) / args.steps,
                         "note": "activations enter as bf16; quantise + pack + send in one kernel; bit-identical output"}
        del layer, x, out_b

    # ---- parity of the layer output against the oracle (every rank, its own tokens)
    rep = layer_parity(oracle, ep, tok_all, weights, shards, world, outs[transports[0]], sl)
    check_layer_parity(rep)
    reports = [None] * world
    if world > 1:
        dist.all_gather_object(reports, rep)
    else:
        reports = [rep]
    del tok_all, outs
    torch.cuda.empty_cache()

    # ---- the same layer call from host buffers: this rank's token tensors come from pinned host memory and its
    # output rows go back to pinned host memory inside the timed region.  The copies run on two more streams (one per
    # direction) with two sets of device buffers, so step k + 1's inputs and step k - 1's output travel while step k
    # computes.
    layer = ep.ExpertParallelMoE(weights, rank, world, transport=transports[0])
    pin = lambda t: t.cpu().pin_memory()
    h_in = [pin(logits), pin(bias), pin(hidden.view(torch.uint8)), pin(hscale)]
    d_in = [[torch.empty_like(logits), torch.empty_like(bias), torch.empty_like(hidden.view(torch.uint8)),
             torch.empty_like(hscale)] for _ in range(2)]
    d_out = [torch.empty((T, H), dtype=torch.bfloat16, device=dev) for _ in range(2)]
    h_out = torch.empty((T, H), dtype=torch.bfloat16).pin_memory()
    copy_stream = torch.cuda.Stream(device=dev)      # host -> device
    back_stream = torch.cuda.Stream(device=dev)      # device -> host: its own stream, so both directions of the link run at once
    main = torch.cuda.current_stream(dev)
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_ready = [torch.cuda.Event() for _ in range(2)]
    out_free = [torch.cuda.Event() for _ in range(2)]

    def upload(k):
        b = k & 1
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(in_free[b])
            for d, hsrc in zip(d_in[b], h_in):
                d.copy_(hsrc, non_blocking=True)
            in_ready[b].record(copy_stream)

    def host_loop(n):
        for ev in in_free + out_free:
            ev.record(main)
        upload(0)
        for k in range(n):
            b = k & 1
            if k + 1 < n:
                upload(k + 1)
            main.wait_event(in_ready[b])
            o = layer.forward(d_in[b][0], d_in[b][1], d_in[b][2].view(torch.float8_e4m3fn), d_in[b][3], RSF)
            main.wait_event(out_free[b])
            d_out[b].copy_(o)
            in_free[b].record(main)
            out_ready[b].record(main)
            with torch.cuda.stream(back_stream):
                back_stream.wait_event(out_ready[b])
                h_out.copy_(d_out[b], non_blocking=True)
                out_free[b].record(back_stream)
        main.wait_stream(copy_stream)
        main.wait_stream(back_stream)

    host_loop(3)
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    host_loop(args.steps)
    e1.record()
    sync()
    ms_host = max_over_ranks(e0.elapsed_time(e1)) / args.steps
    h2d = sum(t.numel() * t.element_size() for t in h_in)
    d2h = h_out.numel() * h_out.element_size()
    del layer
    if rank == 0:
        head = results[transports[0]]
        ms_step, total_rows, rows_max = head["ms_step"], head["rows"], head["rows_max"]
        stage_us = {k: v * 1e3 for k, v in stage_ms.items()}
        if shard_sched is not None:
            g1, g2 = gemm_rooflines(shard_sched, stage_us, P, large=shard_rows > 1024)
            dom = g1 if stage_us["gemm1"] >= stage_us["gemm2"] else g2
            dom["scope"] = (f"one shard call on rank 0 (shard {shards[-1]}, {shard_rows} records, "
                            f"{shard_sched.n_sel} rows)")
            dom["other_gemm"] = g2 if dom is g1 else g1
        else:
            dom = None
        per = 8 // world
        print(json.dumps({
            "metric": METRIC, "value": EP_T / (ms_step * 1e-3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3",
            "data": "synthetic",
            "config": ep_config(world),
            "run_info": {
                "transport": transports[0],
                "dispatch": "one push kernel into the owner's symmetric receive area over NVLink "
                            "(fp8 row + scales + logits per (token, shard))" if transports[0] == "p2p"
                            else "NCCL all_to_all_single",
                "combine": "written by the shard operator's last kernel into the source rank's receive area "
                           "(bf16 row per (token, shard))" if transports[0] == "p2p" else "NCCL all_to_all_single",
                "records_total": total_rows, "records_most_loaded_rank": rows_max,
                "load_balance_bound": total_rows / world / rows_max},
            "gpu_launches": int(head["launches"]),
            "clocks": clocks,
            "bf16_dispatch": bf16_dispatch,
            "nccl_transport": ({"ms_per_step": results["nccl"]["ms_step"],
                                "tokens_per_s": EP_T / (results["nccl"]["ms_step"] * 1e-3)}
                               if "nccl" in results and transports[0] != "nccl" else None),
            "e2e": {"value": EP_T / (ms_host * 1e-3), "unit": UNIT, "ms_per_step": ms_host,
                    "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": d2h * world,
                    "note": "every rank copies its token tensors from pinned host memory and its output rows back; "
                            "copies on two more streams (one per direction), double buffered"},
            "roofline": dom,
            "per_gpu": roofline("whole layer call on the most loaded rank", per * 32 * (W13_BYTES + W2_BYTES),
                                EP_T * 8 * rows_max / total_rows * (FLOPS1 + FLOPS2), ms_step * 1e3, None, P,
                                note="bytes: the rank's weights once; flops: the (token, expert) rows of the most "
                                     "loaded rank, taken as its share of the records times the layer's 8 T rows"),
            "stage_us": stage_us,
            "parity": merge_parity(reports),
            "parity_per_rank": reports,
            "cpu_baseline": None,
        }))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# --impl reference: the definition's CPU path on the host cores, same metric and config
# ---------------------------------------------------------------------------------------------
def bench_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = max(args.gpus, int(os.environ.get("WORLD_SIZE", "1")))
    torch.set_num_threads(os.cpu_count() or 1)      # torchrun exports OMP_NUM_THREADS=1; this arm uses every core
    pkg = load_package()
    gen = pkg.gen
    oracle = load_oracle()
    threads = torch.get_num_threads()
    if world > 1:
        # the 256-expert layer on a bounded token sample: S tokens through all eight shards per step
        S = EP_REFERENCE_SAMPLE
        tok = gen.make_tokens(S, 0, "cpu")      # counter-based generator: the first S tokens of the T-token batch
        cpu_tok = (tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale)
        lazy = [gen.LazyShardWeights(1000 + s, "cpu") for s in range(8)]

        def layer_call():
            acc = None
            for s in range(8):
                o = oracle.run(*cpu_tok, lazy[s].expert, 32 * s, RSF).output.to(torch.float32)
                acc = o if acc is None else acc + o
            return acc.to(torch.bfloat16)
        steps, warmup = min(args.steps, 5), 1
        layer_call()                          # generates the experts the sample uses
        t0 = time.time()
        for _ in range(steps):
            layer_call()
        dt = time.time() - t0
        value = steps * S / dt
        base = {"kind": "port", "cores": threads, "value": value, "unit": UNIT,
                "sample": f"{steps} layer calls of the oracle port on tokens 0..{S - 1} of the T={EP_T} batch, all eight "
                          f"shards, only the experts those tokens use dequantised ({dt:.1f} s)"}
        config, scaling = ep_config(world), "strong"
    else:
        name = args.workload or "decode_t1"
        wl = WORKLOADS[name]
        T = wl["T"]
        tok = gen.make_tokens(T, wl["token_seed"], "cpu", wl["skew"])
        cpu_tok = (tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale)
        definition = load_definition()
        scaling = "weak"
        if definition is not None:
            # the unmodified definition needs the full shard; generate it where that is fastest
            gdev = "cuda" if torch.cuda.is_available() else "cpu"
            W = gen.make_shard_weights(0, gdev)
            cpu_w = [x.cpu() for x in wtuple(W)]
            del W
            steps, warmup = min(args.steps, 3), 1
            definition.run(*cpu_tok, *cpu_w, 0, RSF)
            t0 = time.time()
            for _ in range(steps):
                definition.run(*cpu_tok, *cpu_w, 0, RSF)
            dt = time.time() - t0
            ref = oracle.run_full(*cpu_tok, *cpu_w, 0, RSF)
            kind, what = "reference", "the unmodified definition (all 32 experts dequantised)"
        else:
            lazy = gen.LazyShardWeights(0, "cpu")
            steps, warmup = min(args.steps, 20), min(args.warmup, 3)
            for _ in range(max(1, warmup)):          # also generates the active experts' weights
                oracle.run(*cpu_tok, lazy.expert, 0, RSF)
            t0 = time.time()
            for _ in range(steps):
                ref = oracle.run(*cpu_tok, lazy.expert, 0, RSF)
            dt = time.time() - t0
            kind, what = "port", "the oracle port (only the experts the batch uses dequantised)"
        value = steps * T / dt
        base = {"kind": kind, "cores": threads, "value": value, "unit": UNIT,
                "sample": f"{steps} calls of {what} on the T={T} batch ({dt:.1f} s)"}
        config = workload_config(name, int(ref.counts.sum()), int((ref.counts > 0).sum()))
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "cpu_baseline": base,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------------------------
# The reference's own CUDA solution as the GPU bar (oracle/_ref/libmoe_reference_cuda.so, built by
# oracle/make_ref.py from the unmodified moe.cu): same tensors, same event protocol, its own `run`.
# It runs in a child process so that a fault in it cannot take the measuring process down.
# ---------------------------------------------------------------------------------------------
REF_CUDA_LIB = os.path.join(ROOT, "oracle", "_ref", "libmoe_reference_cuda.so")


def bench_reference_cuda(args):
    """Child leg: times the reference solution's `run` on every single-GPU workload; prints one JSON dict."""
    import tvm_ffi
    pkg = load_package()
    gen = pkg.gen
    oracle = load_oracle()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    mod = tvm_ffi.load_module(REF_CUDA_LIB)
    W = gen.make_shard_weights(0, dev)
    res = {}
    for name, wl in WORKLOADS.items():
        if args.workload and name != args.workload:
            continue
        T = wl["T"]
        tok = gen.make_tokens(T, wl["token_seed"], dev, wl["skew"])
        out = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
        mod.run(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale, *wtuple(W), 0, RSF, out)
        torch.cuda.synchronize()
        _, _, mask = pkg.op.route(tok.routing_logits, tok.routing_bias, 0, RSF)
        used = 0
        for m in mask.cpu().tolist():
            used |= m & 0xFFFFFFFF
        reps = weight_replicas(W, max(1, bin(used).count("1")) * (W13_BYTES + W2_BYTES))
        R = len(reps)

        def step(i=0):
            mod.run(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale,
                    *wtuple(reps[i % R]), 0, RSF, out)
        ms = time_steps(step, 30, 5)
        step(0)
        torch.cuda.synchronize()
        try:
            parity, _ = oracle_check(oracle, tok, W, out, T)
        except AssertionError as e:
            parity = {"failed": str(e)[:300]}
        res[name] = {"us_per_step": ms * 1e3, "tokens_per_s": T / (ms * 1e-3), "parity": parity, "replicas": R}
        del reps
    print("REFERENCE_CUDA " + json.dumps(res))


def reference_cuda_rows():
    """Parent side: run the child leg once and return {workload: row} or {"unavailable": reason}."""
    if not os.path.exists(REF_CUDA_LIB):
        return {"unavailable": "oracle/_ref/libmoe_reference_cuda.so was not built (no reference checkout at build time)"}
    try:
        r = subprocess.run([sys.executable, os.path.abspath(__file__), "--impl", "reference-cuda"], capture_output=True,
                           text=True, timeout=600)
    except subprocess.TimeoutExpired:
        return {"unavailable": "the reference CUDA leg did not finish within 600 s"}
    for ln in r.stdout.splitlines():
        if ln.startswith("REFERENCE_CUDA "):
            return json.loads(ln[len("REFERENCE_CUDA "):])
    return {"unavailable": f"child exited {r.returncode}: {(r.stderr or r.stdout)[-300:]}"}


# sequence lengths of the stand-in trace set (`--replay synthetic`): the five single-GPU configurations plus
# ragged sizes either side of the kernel-path boundaries (16 / 1024 tokens)
REPLAY_SEQ_LENS = (1, 8, 16, 17, 53, 64, 130, 512, 1024, 1025, 4096)


def bench_replay(args):
    """Replays a flashinfer-trace workload set (or a stand-in written on the spot) through the operator with the
    harness's settings, the oracle as the checker, and prints the per-workload table as one JSON line.  When the
    reference's CUDA solution has been built, it is timed on the same tensors as each workload's reference latency."""
    import tempfile
    pkg = load_package()
    oracle = load_oracle()
    rp = pkg.replay
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    root, data = args.replay, "trace set"
    tmp = None
    if root == "synthetic":
        tmp = tempfile.TemporaryDirectory()
        root = tmp.name
        rp.write_synthetic_trace(root, REPLAY_SEQ_LENS, seed=0)
        data = "synthetic stand-in set in the flashinfer-trace layout (routing logits and bias stored, the rest seeded)"
    ref_ms = rp.load_ref_cache(args.ref_cache) if args.ref_cache else {}
    weights = pkg.gen.make_shard_weights(0, dev)
    if not ref_ms and os.path.exists(REF_CUDA_LIB):
        ref_ms = replay_reference_cuda(rp, root, weights, dev)
    res = rp.replay(root, device=dev, checker=oracle.harness_check, ref_latency_ms=ref_ms, weights=weights,
                    limit=args.replay_limit)
    res["replay"] = {"root": args.replay, "data": data, "definition": rp.DEFINITION,
                     "settings": dict(rp.BENCH_DEFAULTS),
                     "ref_latency": ("cache file" if args.ref_cache else
                                     "the reference's CUDA solution timed here on the same tensors" if ref_ms else None)}
    print(json.dumps(res))
    if tmp is not None:
        tmp.cleanup()
    assert res["error"] is None and res["correct"], [(p["axes"], p["status"]) for p in res["per_workload"]]


def replay_reference_cuda(rp, root, weights, dev):
    """{uuid: ms} of the reference's own CUDA solution on every workload of the set (same protocol as ours)."""
    import tvm_ffi
    run = tvm_ffi.load_module(REF_CUDA_LIB).run
    out = {}
    files = {}
    for wl in rp.read_workloads(root):
        if wl.seq_len == 0:
            continue
        try:
            inp = rp.materialise(wl, root, dev, weights=weights, _files=files)
        except rp.TraceError:
            continue
        o = torch.empty(wl.seq_len, H, dtype=torch.bfloat16, device=dev)
        a = [inp[n] for n in rp.INPUT_ORDER] + [o]
        trials = rp.time_workload(lambda: run(*a), dev, rp.BENCH_DEFAULTS["warmup_runs"], rp.BENCH_DEFAULTS["iterations"],
                                  rp.BENCH_DEFAULTS["num_trials"])
        out[wl.uuid] = sum(trials) / len(trials)
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-cuda"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--no-sweep", dest="sweep", action="store_false")
    ap.add_argument("--profile-only", action="store_true",
                    help="run W + K steps of the workload and exit (no checks, no CPU legs): the command profiler "
                         "captures are taken from")
    ap.add_argument("--replay", default=None, metavar="ROOT",
                    help="replay a flashinfer-trace workload set rooted at ROOT ('synthetic': a stand-in set written to "
                         "a temporary directory) and print the per-workload table")
    ap.add_argument("--ref-cache", default=None, help="reference latencies for --replay ({uuid: {ref_latency_ms}})")
    ap.add_argument("--replay-limit", type=int, default=0, help="cap the number of replayed workloads (0 = all)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.replay:
        return bench_replay(args)
    if args.profile_only:
        return profile_only(args)
    if args.impl == "reference":
        return bench_reference(args)
    if args.impl == "reference-cuda":
        return bench_reference_cuda(args)
    if args.gpus > 1 or int(os.environ.get("WORLD_SIZE", "1")) > 1:
        return bench_ep(args)
    return bench_single(args)


if __name__ == "__main__":
    main()
