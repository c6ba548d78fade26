"""CPU tests of the C-ABI boundary: the library loads, exports exactly what
include/moe_b200.h declares, sizes its workspace consistently, and rejects bad
arguments before touching a device.  No compute call is made."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def loader(pkg):
    pkg.build.build()
    return pkg.loader


def declared_functions():
    text = open(os.path.join(ROOT, "include", "moe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(moe_(?:fp8_block_scale|ep)_\w+)\s*\(", text)))


def test_header_and_library_agree(loader):
    names = declared_functions()
    assert len(names) >= 6
    for n in names:
        assert hasattr(loader.lib, n), f"{n} declared in the header but not exported"
    assert sorted(loader.EXPORTS) == names


def test_workspace_size_and_layout(loader):
    prev = 0
    for T in (0, 1, 8, 64, 129, 4096, 16384):
        n = loader.workspace_bytes(T)
        assert n >= prev and n % 256 == 0
        prev = n
        L = loader.layout(T)
        assert L.total == n and L.rows_cap >= 8 * T and L.rows_cap % 128 == 0
        offs = [L.sched, L.topk_idx, L.topk_w, L.local_mask, L.perm_token, L.perm_weight, L.tok_rows,
                L.a_packed, L.a_scale_rows, L.g1, L.cq, L.c_scale, L.o]
        assert offs == sorted(offs) and all(o % 1024 == 0 for o in offs) and offs[-1] < n
    assert loader.workspace_bytes(-1) == 0
    assert ctypes.sizeof(loader.Sched) == (16 + 32 + 33 + 33 + 33) * 4


def test_bad_arguments_are_rejected_without_a_device(loader):
    lib = loader.lib
    fake = 1 << 20        # non-null, 1024-aligned; never dereferenced on these paths
    ok_args = [fake] * 8
    assert lib.moe_fp8_block_scale_run(*ok_args, -1, 0, 2.5, fake, fake, 1 << 40, None) == loader.EINVAL
    assert lib.moe_fp8_block_scale_run(*ok_args, 0, 0, 2.5, fake, fake, 0, None) == loader.OK       # T == 0: no-op
    assert lib.moe_fp8_block_scale_run(None, *ok_args[1:], 4, 0, 2.5, fake, fake, 1 << 40, None) == loader.EINVAL
    assert lib.moe_fp8_block_scale_run(*ok_args, 4, 0, 2.5, fake, fake + 8, 1 << 40, None) == loader.EINVAL  # workspace alignment
    assert lib.moe_fp8_block_scale_run(*ok_args, 4, 0, 2.5, fake, fake, 1024, None) == loader.EWORKSPACE
    assert lib.moe_fp8_block_scale_run_host(*ok_args, 4, 0, 2.5, fake, fake, 1024, None) == loader.EWORKSPACE
    assert lib.moe_fp8_block_scale_layout(-3, None) == loader.EINVAL
    with pytest.raises(loader.MoeLibraryError):
        loader.check(loader.EWORKSPACE)


def test_operator_argument_validation(pkg, loader):
    """The Python mirror of the entry point refuses shapes and dtypes the definition refuses."""
    op = pkg.op
    T = 4
    good = dict(
        routing_logits=torch.zeros(T, 256), routing_bias=torch.zeros(256, dtype=torch.bfloat16),
        hidden_states=torch.zeros(T, 7168).to(torch.float8_e4m3fn), hidden_states_scale=torch.zeros(56, T),
        gemm1_weights=torch.zeros(1, dtype=torch.float8_e4m3fn).expand(32, 4096, 7168),
        gemm1_weights_scale=torch.zeros(32, 32, 56),
        gemm2_weights=torch.zeros(1, dtype=torch.float8_e4m3fn).expand(32, 7168, 2048),
        gemm2_weights_scale=torch.zeros(32, 56, 16), output=torch.zeros(T, 7168, dtype=torch.bfloat16))
    bad = [("routing_logits", torch.zeros(T, 128)), ("routing_bias", torch.zeros(256)),
           ("hidden_states", torch.zeros(T, 7168)), ("hidden_states_scale", torch.zeros(T, 56)),
           ("gemm1_weights_scale", torch.zeros(32, 56, 32)), ("output", torch.zeros(T, 7168))]
    for name, t in bad:
        kw = dict(good)
        kw[name] = t
        with pytest.raises(ValueError):
            op._validate(*[kw[k] for k in ("routing_logits", "routing_bias", "hidden_states", "hidden_states_scale",
                                          "gemm1_weights", "gemm1_weights_scale", "gemm2_weights",
                                          "gemm2_weights_scale", "output")], device_inputs=False)


def test_refused_argument_sets_are_not_remembered(pkg, loader):
    """The wrapper skips the checks for argument sets it has validated before; a set it refused must
    not enter that memory."""
    op = pkg.op
    T = 3
    w13 = torch.zeros(1, dtype=torch.float8_e4m3fn).expand(32, 4096, 7168)
    w2 = torch.zeros(1, dtype=torch.float8_e4m3fn).expand(32, 7168, 2048)

    def make():
        return (torch.zeros(T, 256), torch.zeros(256, dtype=torch.bfloat16), torch.zeros(T, 7168).to(torch.float8_e4m3fn),
                torch.zeros(56, T), w13, torch.zeros(32, 32, 56), w2, torch.zeros(32, 56, 16),
                torch.zeros(T, 7168, dtype=torch.bfloat16))
    op._validated.clear()
    sets = [make() for _ in range(3)]
    for a in sets:
        # (expanded weights are not contiguous: this set is refused, and a refused set is not remembered)
        with pytest.raises(ValueError):
            op._validate(*a, device_inputs=False)
    assert len(op._validated) == 0
    sets = [a[:4] + (torch.zeros(32, 1, 1).to(torch.float8_e4m3fn),) + a[5:6] + (torch.zeros(32, 1, 1).to(torch.float8_e4m3fn),) + a[7:]
            for a in sets]
    for a in sets:
        with pytest.raises(ValueError):      # wrong weight shape
            op._validate(*a, device_inputs=False)
    assert len(op._validated) == 0
