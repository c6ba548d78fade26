"""GPU test of the failure-detection path: a bounded wait that runs out.

Every spin in the kernels (mbarrier waits of the TMA / UMMA pipeline, the decode kernel's grid
barrier) gives up after a time limit, raises a flag and lets the kernel finish normally; the host
reads error bits.  Here a test-only kernel (tests/wait_probe.cu, compiled on the spot with the
limit set to one millisecond) waits for arrivals that never come: the launch must return, the
error bits must be set, and the next ordinary operator call on the same context must be clean."""
import ctypes
import os
import shutil
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def test_bounded_waits_run_out_and_the_context_stays_usable(pkg, tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc is not available to build the probe")
    lib_path = str(tmp_path / "libwait_probe.so")
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", "-shared", "-Xcompiler",
                    "-fPIC", "-I", os.path.join(ROOT, "mlsys-contest-syfi-fully-agent_b200", "csrc"), "-o", lib_path,
                    os.path.join(HERE, "wait_probe.cu")], check=True)
    lib = ctypes.CDLL(lib_path)
    lib.moe_test_wait_timeouts.restype = ctypes.c_int
    lib.moe_test_wait_timeouts.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    dev = torch.device("cuda", 0)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    word = torch.zeros(2, dtype=torch.int32, device=dev)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    assert lib.moe_test_wait_timeouts(status.data_ptr(), word.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    t1.record()
    torch.cuda.synchronize()                       # returns: nothing spins forever
    assert t0.elapsed_time(t1) < 100.0             # two waits of ~1 ms each, not the library's 0.4 s, not a hang
    bits = int(status.item())
    assert bits & 0x1, "the grid-barrier wait did not report its timeout"
    assert bits & 0x2 and bits & 0x200, "the mbarrier wait did not report its timeout / raise the CTA's abort flag"
    assert not bits & 0x100
    # the context is intact: an ordinary call runs and reports no error bits
    gen, op = pkg.gen, pkg.op
    tok = gen.make_tokens(8, 0, dev)
    _, _, mask = op.route(tok.routing_logits, tok.routing_bias, 0, 2.5)
    used = 0
    for m in mask.cpu().tolist():
        used |= m & 0xFFFFFFFF
    W = gen.make_shard_weights(0, dev, experts=[le for le in range(32) if (used >> le) & 1])
    out = op.run(tok.routing_logits, tok.routing_bias, tok.hidden_states, tok.hidden_states_scale, W.gemm1_weights,
                 W.gemm1_weights_scale, W.gemm2_weights, W.gemm2_weights_scale, 0, 2.5)
    assert op.kernel_status() == 0
    assert bool(torch.isfinite(out.float()).all())
