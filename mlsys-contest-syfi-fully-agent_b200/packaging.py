"""Pack the CUDA sources the way the reference solution is packed for the contest harness.

The reference keeps one solution per directory: ``config.toml`` + ``solution/cuda/*`` and a
``solution.json`` that embeds every source file verbatim (moe/config.toml:1-11,
moe/scripts/pack_solution.py:34-86, moe/solution.json).  ``pack(out_dir)`` writes the same three
things for this implementation, with ``entry_point = "tvm_ffi_shim.cu::run"``: the sources of
``csrc/`` plus ``include/moe_b200.h`` flattened into one directory (the harness compiles a flat
list of files), so ``flashinfer_bench`` can load it unchanged.
"""
from __future__ import annotations

import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")

NAME = "b200-moe-fp8-tcgen05"
DEFINITION = "moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048"
AUTHOR = "b200-native"
ENTRY_POINT = "tvm_ffi_shim.cu::run"

SOURCE_FILES = ["tvm_ffi_shim.cu", "launcher.cu", "route_permute.cu", "grouped_gemm.cu", "decode_kernel.cu", "swiglu_combine.cu",
                "static_entry.cu", "quantize.cu", "ep_push.cu", "kernels.h", "moe_layout.h", "ptx.cuh", "route_device.cuh",
                "epilogue_device.cuh", "gemm_common.cuh"]


def flattened_sources():
    """[(file name, content)] with the public header next to the sources."""
    out = []
    for f in SOURCE_FILES:
        text = open(os.path.join(CSRC, f)).read().replace('#include "../../include/moe_b200.h"',
                                                           '#include "moe_b200.h"')
        out.append((f, text))
    out.append(("moe_b200.h", open(os.path.join(ROOT, "include", "moe_b200.h")).read()))
    return out


def solution_dict() -> dict:
    """Same keys as the reference's solution.json."""
    return {
        "name": NAME,
        "definition": DEFINITION,
        "author": AUTHOR,
        "spec": {"language": "cuda", "target_hardware": ["cuda"], "entry_point": ENTRY_POINT,
                 "dependencies": [], "destination_passing_style": True, "binding": None},
        "sources": [{"path": p, "content": c} for p, c in flattened_sources()],
        "description": "FP8 block-scale DeepSeek-V3 MoE shard for sm_100a (tcgen05 / TMA / TMEM).",
    }


CONFIG_TOML = f"""[solution]
name = "{NAME}"
definition = "{DEFINITION}"
author = "{AUTHOR}"

[build]
language = "cuda"
entry_point = "{ENTRY_POINT}"
target_hardware = ["cuda"]
destination_passing_style = true
binding = "tvm-ffi"
"""


def pack(out_dir: str) -> str:
    src_dir = os.path.join(out_dir, "solution", "cuda")
    os.makedirs(src_dir, exist_ok=True)
    for name, text in flattened_sources():
        with open(os.path.join(src_dir, name), "w") as f:
            f.write(text)
    with open(os.path.join(out_dir, "config.toml"), "w") as f:
        f.write(CONFIG_TOML)
    path = os.path.join(out_dir, "solution.json")
    with open(path, "w") as f:
        json.dump(solution_dict(), f, indent=2)
    return path


if __name__ == "__main__":
    import sys
    print(pack(sys.argv[1] if len(sys.argv) > 1 else os.path.join(ROOT, "build", "solution_pack")))
