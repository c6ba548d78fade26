"""CPU tests of the harness packaging: same schema as the reference's solution.json, every
source embedded verbatim, and the flattened directory builds on its own with nvcc + tvm-ffi."""
import json
import os
import subprocess

import pytest

REFERENCE_KEYS = {"name", "definition", "author", "spec", "sources", "description"}
REFERENCE_SPEC_KEYS = {"language", "target_hardware", "entry_point", "dependencies", "destination_passing_style",
                       "binding"}


def test_solution_json_schema(pkg, tmp_path):
    path = pkg.packaging.pack(str(tmp_path))
    d = json.load(open(path))
    assert set(d) == REFERENCE_KEYS and set(d["spec"]) == REFERENCE_SPEC_KEYS
    assert d["definition"] == "moe_fp8_block_scale_ds_routing_topk8_ng8_kg4_e32_h7168_i2048"
    assert d["spec"]["language"] == "cuda" and d["spec"]["destination_passing_style"] is True
    entry_file, entry_fn = d["spec"]["entry_point"].split("::")
    names = [s["path"] for s in d["sources"]]
    assert entry_file in names and entry_fn == "run"
    for s in d["sources"]:
        assert open(tmp_path / "solution" / "cuda" / s["path"]).read() == s["content"]
        assert "../../include" not in s["content"]
    shim = next(s["content"] for s in d["sources"] if s["path"] == entry_file)
    assert "TVM_FFI_DLL_EXPORT_TYPED_FUNC(run" in shim
    toml = open(tmp_path / "config.toml").read()
    assert 'entry_point = "tvm_ffi_shim.cu::run"' in toml and 'binding = "tvm-ffi"' in toml


def test_flattened_directory_compiles(pkg, tmp_path):
    paths = pkg.build.tvmffi_paths()
    if paths is None:
        pytest.skip("tvm-ffi headers not installed")
    pkg.packaging.pack(str(tmp_path))
    src = tmp_path / "solution" / "cuda"
    cus = sorted(str(p) for p in src.glob("*.cu"))
    inc, libdir = paths
    out = tmp_path / "packed.so"
    cmd = [pkg.build._nvcc()] + pkg.build.NVCC_FLAGS + ["-I", inc, "-o", str(out)] + cus + ["-L", libdir, "-ltvm_ffi"]
    subprocess.run(cmd, check=True, cwd=str(src))
    syms = subprocess.run(["nm", "-D", str(out)], check=True, capture_output=True, text=True).stdout
    assert "__tvm_ffi_run" in syms
