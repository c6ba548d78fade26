"""Places the reference's own PyTorch definition of the operator under ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY (like everything under ``oracle/``).  The definition is one Python file
(``full-agent-pipeline/references/moe.py`` of the reference checkout).  It is not part of this
repository: ``oracle/_ref/`` is git-ignored, and this recipe copies the file there UNMODIFIED
from a reference checkout when one is present, so that

* ``bench.py --impl reference`` and the ``cpu_baseline`` leg can time the definition itself
  (``kind: "reference"``: all 32 experts dequantised, as the definition does) instead of the
  oracle port, and
* the benchmark can re-check on the measuring box that the oracle port is bit-identical to it.

``build_reference_cuda`` compiles the reference's CUDA solution (``moe/solution/cuda/moe.cu``, one
file, its own tvm-ffi export) for sm_100a straight from the checkout into
``oracle/_ref/libmoe_reference_cuda.so``: the GPU bar that ``bench.py`` times beside this
repository's kernels.  No reference source is copied for that, only the built library is kept.

Without a reference checkout nothing is written and those legs fall back to the oracle port /
report the GPU bar as unavailable.

    python oracle/make_ref.py [--reference /path/to/reference]
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
DEST_DIR = os.path.join(HERE, "_ref")
DEST = os.path.join(DEST_DIR, "moe_definition.py")
DEFAULT_REFERENCE = os.environ.get("MOE_REFERENCE_ROOT", "/root/reference")   # checkout of the reference repository


def make_ref(reference: str = DEFAULT_REFERENCE):
    """Returns the path of the placed file, or None when no reference checkout is available."""
    src = os.path.join(reference, "full-agent-pipeline", "references", "moe.py")
    if not os.path.exists(src):
        return DEST if os.path.exists(DEST) else None
    os.makedirs(DEST_DIR, exist_ok=True)
    shutil.copyfile(src, DEST)
    with open(DEST, "rb") as f:
        digest = hashlib.sha256(f.read()).hexdigest()
    with open(os.path.join(DEST_DIR, "SOURCE.txt"), "w") as f:
        f.write(f"copied unmodified from {src}\nsha256 {digest}\n")
    return DEST


REF_CUDA_LIB = os.path.join(DEST_DIR, "libmoe_reference_cuda.so")


def build_reference_cuda(reference: str = DEFAULT_REFERENCE):
    """nvcc -arch sm_100a of the unmodified moe.cu + tvm-ffi.  Returns the library path, or None when the
    checkout, nvcc or the tvm-ffi headers are missing (an existing build is kept)."""
    src = os.path.join(reference, "moe", "solution", "cuda", "moe.cu")
    have = REF_CUDA_LIB if os.path.exists(REF_CUDA_LIB) else None
    if not os.path.exists(src):
        return have
    try:
        from tvm_ffi import libinfo
        inc = libinfo.find_include_path()
        libdir = os.path.dirname(libinfo.find_libtvm_ffi())
    except Exception:
        return have
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        return have
    if have and os.path.getmtime(have) >= os.path.getmtime(src):
        return have
    os.makedirs(DEST_DIR, exist_ok=True)
    incs = ["-I", inc]
    for extra in (os.path.join(inc, "..", "3rdparty", "dlpack", "include"),
                  os.path.join(os.path.dirname(inc), "include", "dlpack")):
        if os.path.isdir(extra):
            incs += ["-I", extra]
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-w", "-shared", "-Xcompiler",
           "-fPIC"] + incs + ["-o", REF_CUDA_LIB, src, "-L", libdir, "-ltvm_ffi", "-lcuda", "-Xlinker",
                              "-rpath," + libdir]
    subprocess.run(cmd, check=True)
    return REF_CUDA_LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ref = ap.parse_args().reference
    print(make_ref(ref))
    print(build_reference_cuda(ref))
