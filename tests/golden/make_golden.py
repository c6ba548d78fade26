"""Generate the golden fixtures in this directory from the UNMODIFIED reference definition.

Run once, in a checkout that has the reference mounted:

    python tests/golden/make_golden.py --reference /path/to/reference

For every case it
  1. builds the seeded inputs with the package's generator (full 32-expert shard),
  2. calls ``run`` of ``full-agent-pipeline/references/moe.py`` (imported by path, unmodified),
  3. calls the restated oracle (``oracle/moe_oracle.py``) on the same tensors,
  4. asserts the two bf16 outputs are bit-identical (this is what pins the oracle),
  5. stores selection / permutation / output as ``<case>.npz`` plus input digests.

The fixtures are small: the T=4096 case stores 48 output rows and a digest of the rest.
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys
import time

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from __graft_entry__ import load_package  # noqa: E402

pkg = load_package()
gen = pkg.gen
sys.path.insert(0, os.path.join(ROOT, "oracle"))
import moe_oracle  # noqa: E402

CASES = {
    # name:            T, token seed, skew, local_expert_offset
    "cpu_ref_t8":      dict(T=8, seed=0, skew=False, offset=0),
    "decode_t1":       dict(T=1, seed=None, skew=False, offset=0),     # first seed >= 0 with a local expert
    "skew_t64":        dict(T=64, seed=0, skew=True, offset=0),
    "offset64_t8":     dict(T=8, seed=0, skew=False, offset=64),
    "ragged_t37":      dict(T=37, seed=3, skew=False, offset=0),
    "prefill_t4096":   dict(T=4096, seed=0, skew=False, offset=0),
}
WEIGHT_SEED = 0
SAMPLE_ROWS = 48


def load_reference(path):
    f = os.path.join(path, "full-agent-pipeline", "references", "moe.py")
    spec = importlib.util.spec_from_file_location("reference_moe", f)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def first_seed_with_local_expert(T, skew, offset):
    for seed in range(0, 64):
        tok = gen.make_tokens(T, seed, "cpu", skew)
        idx, _ = moe_oracle.routing(tok.routing_logits, tok.routing_bias, gen.ROUTED_SCALING_FACTOR)
        if ((idx >= offset) & (idx < offset + 32)).any():
            return seed
    raise RuntimeError("no seed found")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference repository")
    ap.add_argument("--cases", default=",".join(CASES))
    args = ap.parse_args()
    ref = load_reference(args.reference)
    torch.manual_seed(0)

    t0 = time.time()
    W = gen.make_shard_weights(WEIGHT_SEED, "cpu")
    wdig = {f"w_expert{le}": gen.digest(W.gemm1_weights[le], W.gemm1_weights_scale[le],
                                        W.gemm2_weights[le], W.gemm2_weights_scale[le]) for le in (0, 5, 31)}
    print(f"weights generated in {time.time() - t0:.0f}s", flush=True)

    for name in args.cases.split(","):
        c = dict(CASES[name])
        if c["seed"] is None:
            c["seed"] = first_seed_with_local_expert(c["T"], c["skew"], c["offset"])
        tok = gen.make_tokens(c["T"], c["seed"], "cpu", c["skew"])
        t0 = time.time()
        out_ref = ref.run(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale,
                          W.gemm1_weights, W.gemm1_weights_scale, W.gemm2_weights, W.gemm2_weights_scale,
                          c["offset"], gen.ROUTED_SCALING_FACTOR)
        t_ref = time.time() - t0
        t0 = time.time()
        orc = moe_oracle.run_full(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale,
                                  W.gemm1_weights, W.gemm1_weights_scale, W.gemm2_weights, W.gemm2_weights_scale,
                                  c["offset"], gen.ROUTED_SCALING_FACTOR)
        t_orc = time.time() - t0
        same = torch.equal(out_ref.view(torch.int16), orc.output.view(torch.int16))
        print(f"{name}: T={c['T']} seed={c['seed']} n_sel={int(orc.counts.sum())} "
              f"active={int((orc.counts > 0).sum())} reference {t_ref:.1f}s oracle {t_orc:.1f}s "
              f"bit-identical={same}", flush=True)
        assert same, "restated oracle differs from the reference definition"

        T = c["T"]
        out_u16 = out_ref.view(torch.int16).numpy().view(np.uint16)
        if T > 256:
            rows = np.unique(np.concatenate([
                np.linspace(0, T - 1, SAMPLE_ROWS // 2).astype(np.int64),
                torch.argsort(orc.output_f32.abs().amax(dim=1), descending=True)[:SAMPLE_ROWS // 2].numpy()]))
        else:
            rows = np.arange(T)
        gap_g, gap_e = moe_oracle.selection_margins(tok.routing_logits, tok.routing_bias)
        meta = dict(case=name, T=T, token_seed=c["seed"], weight_seed=WEIGHT_SEED, skew=c["skew"],
                    local_expert_offset=c["offset"], routed_scaling_factor=gen.ROUTED_SCALING_FACTOR,
                    n_sel=int(orc.counts.sum()), n_active=int((orc.counts > 0).sum()),
                    out_rms=float(orc.output_f32.double().pow(2).mean().sqrt()),
                    out_digest=gen.digest(out_ref),
                    tokens_digest=gen.digest(tok.routing_logits, tok.routing_bias, tok.hidden_states,
                                             tok.hidden_states_scale),
                    weights_digest=wdig, reference_seconds=t_ref, torch=torch.__version__,
                    min_group_gap=float(gap_g.min()), min_expert_gap=float(gap_e.min()))
        np.savez_compressed(
            os.path.join(HERE, name + ".npz"),
            meta=json.dumps(meta),
            topk_sorted=torch.sort(orc.topk_idx, dim=1).values.numpy().astype(np.int16),
            counts=orc.counts.numpy().astype(np.int32),
            offsets=orc.offsets.numpy().astype(np.int32),
            perm_token=orc.perm_token.numpy().astype(np.int32),
            perm_weight=orc.perm_weight.numpy().astype(np.float32),
            rows=rows.astype(np.int32),
            out_bf16=out_u16[rows],
            out_f32=orc.output_f32.numpy()[rows].astype(np.float32),
        )
    print("done")


if __name__ == "__main__":
    main()
