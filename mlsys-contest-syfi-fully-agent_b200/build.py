"""In-tree nvcc build of the CUDA sources for sm_100a.

``build()`` produces ``libmoe_b200.so`` (the C-ABI library declared in
``include/moe_b200.h``) next to this file and, when the tvm-ffi headers are
importable, ``libmoe_b200_tvmffi.so`` (the ``run`` export the contest harness
loads).  Nothing is JIT-compiled at import time elsewhere: the loader refuses
to work without the built library.
"""
from __future__ import annotations

import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libmoe_b200.so")
LIB_TVMFFI = os.path.join(HERE, "libmoe_b200_tvmffi.so")

SOURCES = ["launcher.cu", "route_permute.cu", "grouped_gemm.cu", "grouped_gemm_large.cu", "decode_kernel.cu", "swiglu_combine.cu", "static_entry.cu", "quantize.cu", "ep_push.cu"]
HEADERS = ["kernels.h", "moe_layout.h", "ptx.cuh", "route_device.cuh", "epilogue_device.cuh", "gemm_common.cuh", os.path.join("..", "..", "include", "moe_b200.h")]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC"]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    srcs = [os.path.join(CSRC, s) for s in SOURCES]
    deps = srcs + [os.path.join(CSRC, h) for h in HEADERS] + [os.path.abspath(__file__)]
    if force or _stale(LIB, deps):
        cmd = [_nvcc()] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-o", LIB] + srcs
        subprocess.run(cmd, check=True, cwd=CSRC)
    build_tvmffi(force=force)
    return LIB


def tvmffi_paths():
    """(include dir, library dir) of an installed tvm-ffi, or None."""
    try:
        from tvm_ffi import libinfo
        inc = libinfo.find_include_path()
        lib = os.path.dirname(libinfo.find_libtvm_ffi())
        # dlpack headers ship in a sibling include directory in some wheels
        return inc, lib
    except Exception:
        return None


def build_tvmffi(force: bool = False):
    """The harness-facing shim: same sources plus csrc/tvm_ffi_shim.cu."""
    shim = os.path.join(CSRC, "tvm_ffi_shim.cu")
    paths = tvmffi_paths()
    if paths is None or not os.path.exists(shim):
        return None
    inc, libdir = paths
    srcs = [os.path.join(CSRC, s) for s in SOURCES] + [shim]
    deps = srcs + [os.path.join(CSRC, h) for h in HEADERS]
    if force or _stale(LIB_TVMFFI, deps):
        incs = ["-I", inc]
        dl = os.path.join(os.path.dirname(inc), "include", "dlpack")
        for extra in (os.path.join(inc, "..", "3rdparty", "dlpack", "include"), dl):
            if os.path.isdir(extra):
                incs += ["-I", extra]
        cmd = [_nvcc()] + NVCC_FLAGS + incs + ["-o", LIB_TVMFFI] + srcs + \
              ["-L", libdir, "-ltvm_ffi", "-Xlinker", "-rpath," + libdir]
        subprocess.run(cmd, check=True, cwd=CSRC)
    return LIB_TVMFFI


if __name__ == "__main__":
    import sys
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
