"""Host-side mirror of the reference operator interface.

``run`` takes the eleven arguments of the reference solution's entry point in
the same order and with the same meaning (moe/solution/cuda/moe.cu:2650-2662;
definition full-agent-pipeline/references/moe.py:29-40), destination passing:
the last argument is the pre-allocated bf16 output.  It validates shapes and
dtypes the way the definition asserts them (references/moe.py:66-87) and calls
the C ABI (include/moe_b200.h) on torch's current CUDA stream.  torch is only
used for device memory and streams.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from . import loader

H, I, E_LOCAL, E_GLOBAL, BLOCK = 7168, 2048, 32, 256, 128


class Workspace:
    """Caller-owned scratch memory, grown on demand (the counterpart of the
    reference's process-global ``Workspace``, moe.cu:2511-2589, but per object
    and released with it)."""

    def __init__(self, device=None):
        self.device = torch.device(device if device is not None else "cuda")
        self._buf: Optional[torch.Tensor] = None
        self._base = 0
        self.nbytes = 0

    def reserve(self, T: int):
        need = _ws_bytes.get(T)
        if need is None:
            need = _ws_bytes[T] = loader.workspace_bytes(T)
        if self._buf is None or need > self.nbytes:
            self._buf = torch.empty(need + 1024, dtype=torch.uint8, device=self.device)
            self._base = (-self._buf.data_ptr()) % 1024
            self.nbytes = need
        return self

    @property
    def ptr(self) -> int:
        return self._buf.data_ptr() + self._base

    def view(self, offset: int, nbytes: int) -> torch.Tensor:
        return self._buf[self._base + offset:self._base + offset + nbytes]


_default_ws: Dict[int, Workspace] = {}
_ws_bytes: Dict[int, int] = {}       # workspace size per token count (a library call otherwise)


def _default_workspace(device: torch.device) -> Workspace:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _default_ws:
        _default_ws[idx] = Workspace(torch.device("cuda", idx))
    return _default_ws[idx]


def _check(cond: bool, msg: str):
    if not cond:
        raise ValueError(msg)


_validated: Dict[tuple, bool] = {}     # signatures of argument sets that passed _validate
_VALIDATED_MAX = 64


def _stream_of(dev: torch.device) -> int:
    """Handle of torch's current stream on ``dev``."""
    try:
        return torch._C._cuda_getCurrentRawStream(dev.index if dev.index is not None else torch.cuda.current_device())
    except AttributeError:      # a torch build without the raw getter
        return torch.cuda.current_stream(dev).cuda_stream


class _on_device:
    """``torch.cuda.device(dev)`` only when ``dev`` is not already current (the context manager costs
    more host time than the launch it wraps)."""

    def __init__(self, dev: torch.device):
        self.ctx = None
        if dev.index is not None and dev.index != torch.cuda.current_device():
            self.ctx = torch.cuda.device(dev)

    def __enter__(self):
        if self.ctx is not None:
            self.ctx.__enter__()

    def __exit__(self, *exc):
        if self.ctx is not None:
            self.ctx.__exit__(*exc)


def _validate(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
              gemm2_weights, gemm2_weights_scale, output, device_inputs: bool):
    """Checks the nine tensors the way the definition asserts them; returns (T, their addresses)."""
    T = routing_logits.shape[0]
    # A serving loop calls with the same buffers again and again (or rotates over a few sets): an argument set
    # whose addresses, dtypes and shapes equal a validated one is not inspected a second time (the checks cost
    # more host time than a decode step's launch).
    args = (routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
            gemm2_weights, gemm2_weights_scale, output)
    ptrs = tuple([t.data_ptr() for t in args])
    sig = (device_inputs, ptrs, tuple([(t.dtype, t.shape) for t in args]))
    if sig in _validated:
        return T, ptrs
    _check(routing_logits.dtype == torch.float32 and tuple(routing_logits.shape) == (T, E_GLOBAL),
           "routing_logits must be float32 [T, 256]")
    _check(routing_bias.dtype == torch.bfloat16 and routing_bias.numel() == E_GLOBAL, "routing_bias must be bfloat16 [256]")
    _check(hidden_states.dtype == torch.float8_e4m3fn and tuple(hidden_states.shape) == (T, H),
           "hidden_states must be float8_e4m3fn [T, 7168]")
    _check(hidden_states_scale.dtype == torch.float32 and tuple(hidden_states_scale.shape) == (H // BLOCK, T),
           "hidden_states_scale must be float32 [56, T]")
    _check(gemm1_weights.dtype == torch.float8_e4m3fn and tuple(gemm1_weights.shape) == (E_LOCAL, 2 * I, H),
           "gemm1_weights must be float8_e4m3fn [32, 4096, 7168]")
    _check(gemm1_weights_scale.dtype == torch.float32 and
           tuple(gemm1_weights_scale.shape) == (E_LOCAL, 2 * I // BLOCK, H // BLOCK),
           "gemm1_weights_scale must be float32 [32, 32, 56]")
    _check(gemm2_weights.dtype == torch.float8_e4m3fn and tuple(gemm2_weights.shape) == (E_LOCAL, H, I),
           "gemm2_weights must be float8_e4m3fn [32, 7168, 2048]")
    _check(gemm2_weights_scale.dtype == torch.float32 and
           tuple(gemm2_weights_scale.shape) == (E_LOCAL, H // BLOCK, I // BLOCK),
           "gemm2_weights_scale must be float32 [32, 56, 16]")
    _check(output.dtype == torch.bfloat16 and tuple(output.shape) == (T, H), "output must be bfloat16 [T, 7168]")
    tensors = dict(routing_logits=routing_logits, routing_bias=routing_bias, hidden_states=hidden_states,
                   hidden_states_scale=hidden_states_scale, gemm1_weights=gemm1_weights,
                   gemm1_weights_scale=gemm1_weights_scale, gemm2_weights=gemm2_weights,
                   gemm2_weights_scale=gemm2_weights_scale, output=output)
    for name, t in tensors.items():
        # size-1 dimensions make torch report odd strides for [56, 1]; numel-sized storage is what matters
        _check(t.is_contiguous(), f"{name} must be contiguous")
        on_device = name.startswith("gemm") or device_inputs
        _check(t.is_cuda == on_device, f"{name} must live on the {'GPU' if on_device else 'host'}")
    if len(_validated) >= _VALIDATED_MAX:
        _validated.clear()
    _validated[sig] = True
    return T, ptrs


def run(routing_logits: torch.Tensor, routing_bias: torch.Tensor, hidden_states: torch.Tensor,
        hidden_states_scale: torch.Tensor, gemm1_weights: torch.Tensor, gemm1_weights_scale: torch.Tensor,
        gemm2_weights: torch.Tensor, gemm2_weights_scale: torch.Tensor, local_expert_offset: int,
        routed_scaling_factor: float, output: Optional[torch.Tensor] = None,
        workspace: Optional[Workspace] = None) -> torch.Tensor:
    """The MoE shard, asynchronous on the current CUDA stream.  ``output`` (bf16
    [T, 7168]) is fully overwritten and returned; it is allocated when omitted."""
    if output is None:
        output = torch.empty((routing_logits.shape[0], H), dtype=torch.bfloat16, device=hidden_states.device)
    T, ptrs = _validate(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                        gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, output, device_inputs=True)
    if T == 0:
        return output
    dev = hidden_states.device
    ws = (workspace or _default_workspace(dev)).reserve(T)
    with _on_device(dev):
        rc = loader.lib.moe_fp8_block_scale_run(*ptrs[:8], T, int(local_expert_offset), float(routed_scaling_factor),
                                                ptrs[8], ws.ptr, ws.nbytes, _stream_of(dev))
    if rc:
        loader.check(rc)
    return output


def run_rows(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
             gemm2_weights, gemm2_weights_scale, local_expert_offset: int, routed_scaling_factor: float,
             output_rows: torch.Tensor, workspace: Optional[Workspace] = None) -> None:
    """The operator with a per-token destination: ``output_rows`` is an int64 CUDA tensor of T device
    addresses (16-byte aligned, 7168 bf16 each; peer-mapped memory allowed) that row t is written to."""
    T = routing_logits.shape[0]
    dummy = torch.empty((T, H), dtype=torch.bfloat16, device="meta")
    _check(output_rows.dtype == torch.int64 and output_rows.numel() == T and output_rows.is_cuda and
           output_rows.is_contiguous(), "output_rows must be a contiguous CUDA int64 tensor of T addresses")
    del dummy
    if T == 0:
        return
    dev = hidden_states.device
    ws = (workspace or _default_workspace(dev)).reserve(T)
    with torch.cuda.device(dev):
        stream = torch.cuda.current_stream(dev).cuda_stream
        rc = loader.lib.moe_fp8_block_scale_run_rows(
            routing_logits.data_ptr(), routing_bias.data_ptr(), hidden_states.data_ptr(),
            hidden_states_scale.data_ptr(), gemm1_weights.data_ptr(), gemm1_weights_scale.data_ptr(),
            gemm2_weights.data_ptr(), gemm2_weights_scale.data_ptr(), int(T), int(local_expert_offset),
            float(routed_scaling_factor), output_rows.data_ptr(), ws.ptr, ws.nbytes, stream)
    loader.check(rc)


def run_host(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights, gemm1_weights_scale,
             gemm2_weights, gemm2_weights_scale, local_expert_offset: int, routed_scaling_factor: float,
             output: torch.Tensor, workspace: Optional[Workspace] = None) -> torch.Tensor:
    """Same operator for token-side tensors in (pinned) host memory: copies them
    in, runs, copies ``output`` (a host tensor) back and waits."""
    T, ptrs = _validate(routing_logits, routing_bias, hidden_states, hidden_states_scale, gemm1_weights,
                        gemm1_weights_scale, gemm2_weights, gemm2_weights_scale, output, device_inputs=False)
    if T == 0:
        return output
    dev = gemm1_weights.device
    ws = (workspace or _default_workspace(dev)).reserve(T)
    with _on_device(dev):
        rc = loader.lib.moe_fp8_block_scale_run_host(*ptrs[:8], T, int(local_expert_offset),
                                                     float(routed_scaling_factor), ptrs[8], ws.ptr, ws.nbytes,
                                                     _stream_of(dev))
    if rc:
        loader.check(rc)
    return output


def route(routing_logits: torch.Tensor, routing_bias: torch.Tensor, local_expert_offset: int,
          routed_scaling_factor: float):
    """Routing alone: (topk_idx i32 [T,8], topk_w f32 [T,8], local_mask i32 [T]) on the current stream."""
    T = routing_logits.shape[0]
    dev = routing_logits.device
    idx = torch.empty((T, 8), dtype=torch.int32, device=dev)
    w = torch.empty((T, 8), dtype=torch.float32, device=dev)
    mask = torch.empty((T,), dtype=torch.int32, device=dev)
    if T:
        with torch.cuda.device(dev):
            loader.check(loader.lib.moe_fp8_block_scale_route(
                routing_logits.data_ptr(), routing_bias.data_ptr(), int(T), int(local_expert_offset),
                float(routed_scaling_factor), idx.data_ptr(), w.data_ptr(), mask.data_ptr(),
                torch.cuda.current_stream(dev).cuda_stream))
    return idx, w, mask


def quantize_activations(hidden_bf16: torch.Tensor):
    """bf16 [T, 7168] -> (e4m3 [T, 7168], fp32 scales [56, T]) in the operator's input layout."""
    _check(hidden_bf16.dtype == torch.bfloat16 and hidden_bf16.dim() == 2 and hidden_bf16.shape[1] == H and
           hidden_bf16.is_contiguous() and hidden_bf16.is_cuda, "hidden must be a contiguous CUDA bfloat16 [T, 7168]")
    T = hidden_bf16.shape[0]
    dev = hidden_bf16.device
    q = torch.empty((T, H), dtype=torch.float8_e4m3fn, device=dev)
    s = torch.empty((H // BLOCK, T), dtype=torch.float32, device=dev)
    if T:
        with torch.cuda.device(dev):
            loader.check(loader.lib.moe_fp8_block_scale_quantize_activations(
                hidden_bf16.data_ptr(), int(T), q.data_ptr(), s.data_ptr(), torch.cuda.current_stream(dev).cuda_stream))
    return q, s


def kernel_status(workspace: Optional[Workspace] = None, device=None) -> int:
    """Waits for the current stream and returns the kernels' error bits (0 = none)."""
    dev = torch.device(device if device is not None else "cuda")
    ws = workspace or _default_workspace(dev)
    st = ctypes.c_int(0)
    with torch.cuda.device(ws.device):
        rc = loader.lib.moe_fp8_block_scale_status(ws.ptr, torch.cuda.current_stream().cuda_stream, ctypes.byref(st))
    if rc not in (loader.OK, loader.EKERNEL):
        loader.check(rc)
    return st.value


def read_schedule(T: int, workspace: Optional[Workspace] = None, device=None) -> "loader.Sched":
    """Waits for the device and returns a host copy of the schedule block the last call with ``T``
    tokens left in the workspace: error bits, rows, active experts, tile widths and split-K factors
    the device chose, per-expert counts and offsets (``include/moe_b200.h``: ``moe_b200_sched``)."""
    dev = torch.device(device if device is not None else "cuda")
    ws = workspace or _default_workspace(dev)
    torch.cuda.synchronize(ws.device)
    L = loader.layout(T)
    raw = ws.view(L.sched, ctypes.sizeof(loader.Sched)).cpu().numpy().tobytes()
    return loader.Sched.from_buffer_copy(raw)
