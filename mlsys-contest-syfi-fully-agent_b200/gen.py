"""Seeded synthetic inputs for the FP8 block-scale DeepSeek-V3 MoE shard.

The contest dataset that the reference is evaluated on is not redistributable
here, so every workload is synthetic: the shapes, dtypes and value
distributions follow the operator definition
(full-agent-pipeline/references/moe.py:29-40 for the signature,
:95-118 for the block-scale layout).

The generator is *counter based*: element ``i`` of tensor stream ``s`` under
seed ``k`` is a pure function of ``(k, s, i)`` built from 64-bit integer
hashing and IEEE float64/float32 arithmetic only.  The same torch code
therefore produces byte-identical tensors on a CPU and on a GPU, and one
expert's weights can be generated without generating the other 31 (the CPU
test-suite relies on that: a full shard is 1.4 G elements).

Approximate normals: the sum of four 16-bit uniform chunks of one hash
(Irwin-Hall, support +-3.46 sigma) plus a 32-bit uniform dither from a second
hash, so that values have ~2^50 distinct levels and exact ties between routing
scores do not occur in practice.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, Optional

import torch

H = 7168            # hidden size
I = 2048            # intermediate size
E_LOCAL = 32        # experts per shard
E_GLOBAL = 256      # experts per layer
BLOCK = 128         # quantisation block
TOP_K = 8
N_GROUP = 8
TOPK_GROUP = 4
FP8_MAX = 448.0

# tensor stream ids
_S_LOGITS, _S_BIAS, _S_HIDDEN, _S_W13, _S_W2 = 1, 2, 3, 4, 5

_M64 = (1 << 64) - 1


def _i64(x: int) -> int:
    """Two's-complement int64 view of an unsigned 64-bit constant."""
    x &= _M64
    return x - (1 << 64) if x >= (1 << 63) else x


_GOLD = _i64(0x9E3779B97F4A7C15)
_MUL1 = _i64(0xBF58476D1CE4E5B9)
_MUL2 = _i64(0x94D049BB133111EB)


def _lsr(z: torch.Tensor, n: int) -> torch.Tensor:
    """Logical shift right of an int64 tensor."""
    return (z >> n) & ((1 << (64 - n)) - 1)


def _mix64(z: torch.Tensor) -> torch.Tensor:
    """splitmix64 finaliser on an int64 tensor (wrapping arithmetic)."""
    z = (z ^ _lsr(z, 30)) * _MUL1
    z = (z ^ _lsr(z, 27)) * _MUL2
    return z ^ _lsr(z, 31)


def _stream_key(seed: int, stream: int, sub: int) -> int:
    k = (seed * 0x9E3779B97F4A7C15 + stream * 0xD1B54A32D192ED03 + sub * 0x8CB92BA72F3D8DD7) & _M64
    # one scalar mix so that nearby seeds do not give shifted copies
    k ^= k >> 30
    k = (k * 0xBF58476D1CE4E5B9) & _M64
    k ^= k >> 27
    k = (k * 0x94D049BB133111EB) & _M64
    k ^= k >> 31
    return _i64(k)


_IH_SIGMA = (4.0 * (65536.0 ** 2 - 1.0) / 12.0) ** 0.5   # std of the 4-chunk sum


def normal(seed: int, stream: int, start: int, count: int, device, chunk: int = 1 << 24) -> torch.Tensor:
    """``count`` approximately-N(0,1) float32 values for flat indices
    ``start .. start+count`` of a stream.  Bit-reproducible on any device."""
    out = torch.empty(count, dtype=torch.float32, device=device)
    ka = _stream_key(seed, stream, 0)
    kb = _stream_key(seed, stream, 1)
    scale = 1.0 / (4294967296.0 * _IH_SIGMA)
    for c0 in range(0, count, chunk):
        n = min(chunk, count - c0)
        idx = torch.arange(start + c0, start + c0 + n, dtype=torch.int64, device=device)
        h1 = _mix64(idx * _GOLD + ka)
        h2 = _mix64(idx * _GOLD + kb)
        s = (h1 & 0xFFFF) + (_lsr(h1, 16) & 0xFFFF) + (_lsr(h1, 32) & 0xFFFF) + _lsr(h1, 48)
        v = (s - 131070) * 4294967296 + (_lsr(h2, 32) - 2147483648)     # |v| < 2^50: exact in float64
        out[c0:c0 + n] = (v.to(torch.float64) * scale).to(torch.float32)
    return out


def _div_ieee(x: torch.Tensor, d: float) -> torch.Tensor:
    """x / d with a correctly rounded division on every device (CUDA turns division by a
    Python scalar into a multiplication by its reciprocal, which differs in the last bit)."""
    return x / torch.full_like(x, d)


def quant_1x128(x: torch.Tensor):
    """Per-row 1x128 block quantisation of ``x`` [R, C] (C % 128 == 0) to e4m3.
    Returns (q fp8 [R, C], scale fp32 [R, C/128]), scale = amax/448."""
    R, C = x.shape
    xb = x.view(R, C // BLOCK, BLOCK)
    amax = xb.abs().amax(dim=2).clamp_min(1e-10)
    scale = _div_ieee(amax, FP8_MAX)
    q = (xb / scale.unsqueeze(2)).to(torch.float8_e4m3fn).view(R, C)
    return q, scale


def quant_128x128(w: torch.Tensor):
    """128x128 block quantisation of ``w`` [R, C] to e4m3.
    Returns (q fp8 [R, C], scale fp32 [R/128, C/128])."""
    R, C = w.shape
    wb = w.view(R // BLOCK, BLOCK, C // BLOCK, BLOCK)
    amax = wb.abs().amax(dim=(1, 3)).clamp_min(1e-10)
    scale = _div_ieee(amax, FP8_MAX)
    q = (wb / scale[:, None, :, None]).to(torch.float8_e4m3fn).view(R, C)
    return q, scale


@dataclass
class TokenInputs:
    """Per-call token-side tensors of the operator."""
    routing_logits: torch.Tensor        # [T, 256] fp32
    routing_bias: torch.Tensor          # [256] bf16
    hidden_states: torch.Tensor         # [T, 7168] e4m3
    hidden_states_scale: torch.Tensor   # [56, T] fp32 (transposed, as the definition wants)


def make_tokens(T: int, seed: int, device="cpu", skew: bool = False) -> TokenInputs:
    """Token-side inputs.  ``skew`` adds +4.0 to the bias of global experts
    0..15 (the load-imbalance workload)."""
    logits = normal(seed, _S_LOGITS, 0, T * E_GLOBAL, device).view(T, E_GLOBAL)
    bias = normal(seed, _S_BIAS, 0, E_GLOBAL, device) * 0.1
    if skew:
        bias[:16] += 4.0
    bias = bias.to(torch.bfloat16)
    hid = normal(seed, _S_HIDDEN, 0, T * H, device).view(T, H).to(torch.bfloat16).to(torch.float32)
    q, sc = quant_1x128(hid)
    return TokenInputs(logits.contiguous(), bias.contiguous(), q.contiguous(), sc.t().contiguous())


def make_expert_weights(seed: int, le: int, device="cpu"):
    """Weights of local expert ``le`` of the shard with weight seed ``seed``:
    (w13 e4m3 [4096,7168], s13 fp32 [32,56], w2 e4m3 [7168,2048], s2 fp32 [56,16])."""
    n13 = 2 * I * H
    w13 = normal(seed, _S_W13, le * n13, n13, device).view(2 * I, H) * 0.02
    q13, s13 = quant_128x128(w13)
    del w13
    n2 = H * I
    w2 = normal(seed, _S_W2, le * n2, n2, device).view(H, I) * 0.02
    q2, s2 = quant_128x128(w2)
    return q13, s13, q2, s2


@dataclass
class ShardWeights:
    """Weights of one 32-expert shard (full tensors, as the operator takes them)."""
    gemm1_weights: torch.Tensor         # [32, 4096, 7168] e4m3
    gemm1_weights_scale: torch.Tensor   # [32, 32, 56] fp32
    gemm2_weights: torch.Tensor         # [32, 7168, 2048] e4m3
    gemm2_weights_scale: torch.Tensor   # [32, 56, 16] fp32


def make_shard_weights(seed: int, device="cpu", experts: Optional[Iterable[int]] = None) -> ShardWeights:
    """All 32 experts of a shard.  With ``experts`` given, only those are
    generated and the others are left zero (cheap CPU tests)."""
    w13 = torch.zeros((E_LOCAL, 2 * I, H), dtype=torch.float8_e4m3fn, device=device)
    s13 = torch.zeros((E_LOCAL, 2 * I // BLOCK, H // BLOCK), dtype=torch.float32, device=device)
    w2 = torch.zeros((E_LOCAL, H, I), dtype=torch.float8_e4m3fn, device=device)
    s2 = torch.zeros((E_LOCAL, H // BLOCK, I // BLOCK), dtype=torch.float32, device=device)
    for le in (range(E_LOCAL) if experts is None else experts):
        a, b, c, d = make_expert_weights(seed, le, device)
        w13[le], s13[le], w2[le], s2[le] = a, b, c, d
    return ShardWeights(w13, s13, w2, s2)


class LazyShardWeights:
    """Per-expert weight access that generates an expert on first use.
    Lets a CPU checker touch only the experts a small batch actually routes to."""

    def __init__(self, seed: int, device="cpu"):
        self.seed, self.device = seed, device
        self._cache: Dict[int, tuple] = {}

    def expert(self, le: int):
        if le not in self._cache:
            self._cache[le] = make_expert_weights(self.seed, le, self.device)
        return self._cache[le]


def digest(*tensors: torch.Tensor) -> str:
    """sha256 over the raw bytes of the tensors (device independent)."""
    import hashlib
    h = hashlib.sha256()
    for t in tensors:
        h.update(t.detach().cpu().reshape(-1).clone().view(torch.uint8).numpy().tobytes())
    return h.hexdigest()


ROUTED_SCALING_FACTOR = 2.5
