"""Test-only readers of the operator's workspace: host copies of the selection, the permutation
and the per-stage arrays that the last call left behind, for the parity tests."""
import ctypes

import torch

H, I = 7168, 2048


def _sum_slabs(arr, offset, sched, gemm, pad, width):
    """fp32 result [pad, width] of one GEMM from its split-K slabs.  General path: `split` equal slabs.
    Decode path (split == 0): a weight-row tile has as many slabs as the balanced partition cut it into
    pieces (csrc/decode_kernel.cu: stage_owner / tile_pieces), computed here from the tile index alone."""
    split = sched.split1 if gemm == 1 else sched.split2
    if split > 0:
        s = arr(offset, split * pad * width * 4, torch.float32, (split, pad, width))
        return s.sum(dim=0) if split > 1 else s[0]
    n, mt = sched.ctas, width // 128
    u = (56 if gemm == 1 else 16) // 2                 # pipeline stages per tile
    G = sched.tiles_total * mt * u
    owner = lambda g: ((g + 1) * n - 1) // G
    pieces = lambda tau: owner(tau * u + u - 1) - owner(tau * u) + 1
    counts, offs = list(sched.counts), list(sched.offs)
    active = [e for e in range(32) if counts[e] > 0]
    smax = max(pieces(t) for t in range(len(active) * mt))
    s = arr(offset, smax * pad * width * 4, torch.float32, (smax, pad, width))
    res = torch.zeros(pad, width, dtype=torch.float32, device=s.device)
    for ordinal, e in enumerate(active):
        rows = slice(offs[e], offs[e + 1])
        for m in range(mt):
            cols = slice(m * 128, (m + 1) * 128)
            for k in range(pieces(ordinal * mt + m)):   # slab order, as the kernel sums
                res[rows, cols] += s[k, rows, cols]
    return res


def intermediates(pkg, T: int, workspace=None, device=None, stages: bool = True) -> dict:
    """Host copies of the selection / permutation / per-stage arrays the last
    call with ``T`` tokens left in the workspace.  ``stages=False`` skips the fp32 / fp8 per-stage
    arrays (hundreds of megabytes for large batches)."""
    op, loader = pkg.op, pkg.loader
    dev = torch.device(device if device is not None else "cuda")
    ws = workspace or op._default_workspace(dev)
    torch.cuda.synchronize(ws.device)
    L = loader.layout(T)

    def arr(off, nbytes, dtype, shape):
        return ws.view(off, nbytes).view(dtype).reshape(shape)

    sched_raw = ws.view(L.sched, ctypes.sizeof(loader.Sched)).cpu().numpy().tobytes()
    sched = loader.Sched.from_buffer_copy(sched_raw)
    n_sel, pad = sched.n_sel, sched.n_sel_pad
    out = dict(
        sched=sched, layout=L, n_sel=n_sel,
        counts=torch.tensor(list(sched.counts)), offs=torch.tensor(list(sched.offs)),
        topk_idx=arr(L.topk_idx, T * 8 * 4, torch.int32, (T, 8)).cpu(),
        topk_w=arr(L.topk_w, T * 8 * 4, torch.float32, (T, 8)).cpu(),
        local_mask=arr(L.local_mask, T * 4, torch.int32, (T,)).cpu(),
        perm_token=arr(L.perm_token, n_sel * 4, torch.int32, (n_sel,)).cpu(),
        perm_weight=arr(L.perm_weight, n_sel * 4, torch.float32, (n_sel,)).cpu(),
        tok_rows=arr(L.tok_rows, T * 8 * 4, torch.int32, (T, 8)).cpu(),
    )
    if n_sel > 0 and stages:
        out["g1"] = _sum_slabs(arr, L.g1, sched, 1, pad, 4096)[:n_sel].cpu()
        out["o"] = _sum_slabs(arr, L.o, sched, 2, pad, H)[:n_sel].cpu()
        cq = arr(L.cq, L.n_terms * L.rows_cap * I, torch.float8_e4m3fn, (L.n_terms, L.rows_cap, I))[:, :n_sel]
        cs = arr(L.c_scale, L.rows_cap * 16 * 4, torch.float32, (L.rows_cap, 16))[:n_sel]
        c = cq.to(torch.float32).sum(dim=0).view(n_sel, 16, 128) * cs.unsqueeze(2)
        out["c"] = c.view(n_sel, I).cpu()
        out["a_packed"] = arr(L.a_packed, n_sel * H, torch.uint8, (n_sel, H)).cpu()
    return out


def swiglu_planes(pkg, T: int, workspace=None, device=None):
    """The SwiGLU output as GEMM2 reads it, left by the last call with ``T`` tokens: (planes u8 [3, n_sel, 2048],
    scales f32 [n_sel, 16]) on the device."""
    op, loader = pkg.op, pkg.loader
    dev = torch.device(device if device is not None else "cuda")
    ws = workspace or op._default_workspace(dev)
    torch.cuda.synchronize(ws.device)
    L = loader.layout(T)
    n_sel = op.read_schedule(T, workspace, device).n_sel
    cq = ws.view(L.cq, L.n_terms * L.rows_cap * I).view(L.n_terms, L.rows_cap, I)[:, :n_sel].clone()
    cs = ws.view(L.c_scale, L.rows_cap * 16 * 4).view(torch.float32).view(L.rows_cap, 16)[:n_sel].clone()
    return cq, cs
