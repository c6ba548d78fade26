"""B200-native FP8 block-scale DeepSeek-V3 MoE shard
(``moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048``).

The directory name is not a Python identifier; load it with
``__graft_entry__.load_package()`` which registers it as ``moe_b200``.

Sub-modules:
  gen     seeded synthetic workloads
  loader  ctypes binding of the C-ABI library (fails loudly if it is missing)
  op      ``run(...)`` with the reference entry point's argument list
  ep      expert-parallel 256-expert layer over torch.distributed
  build   nvcc build of csrc/ for sm_100a
  packaging  config.toml + solution.json in the reference's schema
  replay  a flashinfer-trace workload set run through ``op.run`` (per-workload status, latency, speed-up)
"""
from . import gen  # noqa: F401


def __getattr__(name):
    # torch-free / CUDA-free modules are imported eagerly above; the ones that
    # need the compiled library are resolved on first use.
    if name in ("loader", "op", "ep", "build", "packaging", "replay"):
        import importlib
        return importlib.import_module(f"{__name__}.{name}")
    raise AttributeError(name)
