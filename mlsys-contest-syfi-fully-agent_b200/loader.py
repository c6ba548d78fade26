"""ctypes binding of the C-ABI library (include/moe_b200.h).

There is no fallback: if ``libmoe_b200.so`` has not been built
(``python -m`` of ``build.py`` or ``__graft_entry__.build()``), importing
this module raises.
"""
from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MOE_B200_LIB") or os.path.join(HERE, "libmoe_b200.so")   # override: debug builds

OK, EINVAL, EWORKSPACE, ECUDA, EDEVICE, EKERNEL = 0, -1, -2, -3, -4, -5
ERROR_NAMES = {OK: "ok", EINVAL: "invalid argument", EWORKSPACE: "workspace too small", ECUDA: "CUDA error",
               EDEVICE: "device is not sm_100", EKERNEL: "kernel reported an error"}

EXPORTS = [
    "moe_fp8_block_scale_workspace_bytes",
    "moe_fp8_block_scale_run",
    "moe_fp8_block_scale_run_host",
    "moe_fp8_block_scale_status",
    "moe_fp8_block_scale_last_cuda_error",
    "moe_fp8_block_scale_layout",
    "moe_fp8_block_scale_launch_count",
    "moe_fp8_block_scale_set_profiling",
    "moe_fp8_block_scale_stage_times",
    "moe_fp8_block_scale_route_static",
    "moe_fp8_block_scale_route",
    "moe_fp8_block_scale_quantize_activations",
    "moe_fp8_block_scale_run_rows",
    "moe_fp8_block_scale_set_options",
    "moe_fp8_block_scale_get_options",
    "moe_ep_dispatch_push",
    "moe_ep_sum_shards",
    "moe_ep_plan",
    "moe_ep_row_pointers",
    "moe_ep_quantize_push",
]
STATIC_MAX_TOKENS = 4096
STAGES = ("route_permute", "gather", "gemm1", "swiglu_split", "gemm2", "combine")


class Layout(ctypes.Structure):
    _fields_ = [("T", ctypes.c_int32), ("rows_cap", ctypes.c_int32), ("slab_rows", ctypes.c_int32),
                ("n_terms", ctypes.c_int32)] + \
               [(n, ctypes.c_uint64) for n in ("sched", "topk_idx", "topk_w", "local_mask", "perm_token",
                                               "perm_weight", "tok_rows", "a_packed", "a_scale_rows", "g1", "cq", "c_scale", "o",
                                               "acc32", "tile_cnt", "total")]


class Sched(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("status", "n_sel", "n_sel_pad", "n_active", "n_tile", "tiles_total",
                                              "split1", "split2", "items1", "items2")] + \
               [("bar1", ctypes.c_uint32 * 2), ("bar2", ctypes.c_uint32 * 2), ("n_tile2", ctypes.c_int32), ("ctas", ctypes.c_int32), ("counts", ctypes.c_int32 * 32), ("offs", ctypes.c_int32 * 33),
                ("tile_prefix", ctypes.c_int32 * 33), ("tile_prefix2", ctypes.c_int32 * 33)]


class EpSegment(ctypes.Structure):
    _fields_ = [("first_record", ctypes.c_int64), ("count", ctypes.c_int64), ("dst_hidden", ctypes.c_void_p),
                ("dst_scale", ctypes.c_void_p), ("dst_logits", ctypes.c_void_p)]


class MoeLibraryError(RuntimeError):
    def __init__(self, code: int, cuda_error: int = 0):
        self.code, self.cuda_error = code, cuda_error
        msg = ERROR_NAMES.get(code, f"error {code}")
        if code == ECUDA:
            msg += f" (cudaError {cuda_error})"
        super().__init__(msg)


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it first (python __graft_entry__.py build); "
                          "there is no non-CUDA fallback")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i32, f32, sz = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t
    lib.moe_fp8_block_scale_workspace_bytes.restype = sz
    lib.moe_fp8_block_scale_workspace_bytes.argtypes = [i32]
    run_args = [vp] * 8 + [i32, i32, f32, vp, vp, sz, vp]
    lib.moe_fp8_block_scale_run.restype = i32
    lib.moe_fp8_block_scale_run.argtypes = run_args
    lib.moe_fp8_block_scale_run_host.restype = i32
    lib.moe_fp8_block_scale_run_host.argtypes = run_args
    lib.moe_fp8_block_scale_status.restype = i32
    lib.moe_fp8_block_scale_status.argtypes = [vp, vp, ctypes.POINTER(i32)]
    lib.moe_fp8_block_scale_last_cuda_error.restype = i32
    lib.moe_fp8_block_scale_last_cuda_error.argtypes = []
    lib.moe_fp8_block_scale_layout.restype = i32
    lib.moe_fp8_block_scale_layout.argtypes = [i32, ctypes.POINTER(Layout)]
    lib.moe_fp8_block_scale_route_static.restype = i32
    lib.moe_fp8_block_scale_route_static.argtypes = [vp, vp, i32, i32, f32, vp, vp, vp, vp, vp, vp]
    lib.moe_fp8_block_scale_route.restype = i32
    lib.moe_fp8_block_scale_route.argtypes = [vp, vp, i32, i32, f32, vp, vp, vp, vp]
    lib.moe_fp8_block_scale_quantize_activations.restype = i32
    lib.moe_fp8_block_scale_quantize_activations.argtypes = [vp, i32, vp, vp, vp]
    lib.moe_fp8_block_scale_run_rows.restype = i32
    lib.moe_fp8_block_scale_run_rows.argtypes = run_args
    lib.moe_ep_dispatch_push.restype = i32
    lib.moe_ep_dispatch_push.argtypes = [vp, vp, vp, i32, vp, i32, ctypes.POINTER(EpSegment), i32, vp]
    lib.moe_ep_sum_shards.restype = i32
    lib.moe_ep_sum_shards.argtypes = [vp, vp, i32, vp, vp]
    lib.moe_ep_plan.restype = i32
    lib.moe_ep_plan.argtypes = [vp, i32, vp, vp, vp, vp, vp]
    lib.moe_ep_quantize_push.restype = i32
    lib.moe_ep_quantize_push.argtypes = [vp, vp, i32, vp, ctypes.POINTER(EpSegment), vp]
    lib.moe_ep_row_pointers.restype = i32
    lib.moe_ep_row_pointers.argtypes = [vp, vp, i32, ctypes.c_int64, vp, i32, vp]
    lib.moe_fp8_block_scale_set_options.restype = i32
    lib.moe_fp8_block_scale_set_options.argtypes = [ctypes.c_uint]
    lib.moe_fp8_block_scale_get_options.restype = ctypes.c_uint
    lib.moe_fp8_block_scale_get_options.argtypes = []
    lib.moe_fp8_block_scale_launch_count.restype = ctypes.c_longlong
    lib.moe_fp8_block_scale_launch_count.argtypes = []
    lib.moe_fp8_block_scale_set_profiling.restype = i32
    lib.moe_fp8_block_scale_set_profiling.argtypes = [i32]
    lib.moe_fp8_block_scale_stage_times.restype = i32
    lib.moe_fp8_block_scale_stage_times.argtypes = [ctypes.POINTER(f32), i32]
    return lib


lib = _load()


OPT_FAST_COMBINE, OPT_UNFUSED = 1, 2


def set_options(options: int):
    """Process-wide operator options (include/moe_b200.h: MOE_B200_OPT_*)."""
    check(lib.moe_fp8_block_scale_set_options(int(options)))


def get_options() -> int:
    return int(lib.moe_fp8_block_scale_get_options())


def launch_count() -> int:
    return int(lib.moe_fp8_block_scale_launch_count())


def set_profiling(enable: bool):
    check(lib.moe_fp8_block_scale_set_profiling(1 if enable else 0))


def stage_times_ms() -> dict:
    buf = (ctypes.c_float * len(STAGES))()
    check(lib.moe_fp8_block_scale_stage_times(buf, len(STAGES)))
    return dict(zip(STAGES, [float(x) for x in buf]))


def check(code: int):
    if code != OK:
        raise MoeLibraryError(code, lib.moe_fp8_block_scale_last_cuda_error())


def workspace_bytes(T: int) -> int:
    return int(lib.moe_fp8_block_scale_workspace_bytes(int(T)))


def layout(T: int) -> Layout:
    out = Layout()
    check(lib.moe_fp8_block_scale_layout(int(T), ctypes.byref(out)))
    return out
