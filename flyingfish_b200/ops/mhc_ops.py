"""Manifold-constrained hyper-connections: mixer coefficients (with the Sinkhorn-normalised combination
matrix), stream collapse and residual update. CUDA: ``csrc/mhc.cu``; CPU: FP32 oracles with the same
rounding points (reference: kernels/mhc.cu:1-37, 60-170, 300-438)."""
from __future__ import annotations

from ctypes import c_float

import torch

from . import _count, _require
from .lib import check, kernels, ptr, stream_ptr

BF16 = torch.bfloat16


def mixes(stream: torch.Tensor, fn: torch.Tensor, base: torch.Tensor, scale: torch.Tensor, iters: int, eps: float,
          norm_eps: float) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """stream [rows, mult, hidden] bf16, fn [(2+mult)*mult, mult*hidden] bf16, base [(2+mult)*mult] f32,
    scale [3] f32 -> pre [rows, mult], post [rows, mult], comb [rows, mult, mult] (rows = out, cols = in)."""
    rows, mult, hidden = stream.shape
    if not stream.is_cuda:
        x = stream.float().reshape(rows, mult * hidden)
        r = torch.rsqrt((x * x).mean(1) + norm_eps)
        mix = (x @ fn.float().t()) * r[:, None]
        pre = torch.sigmoid(mix[:, :mult] * scale[0] + base[:mult]) + eps
        post = 2.0 * torch.sigmoid(mix[:, mult: 2 * mult] * scale[1] + base[mult: 2 * mult])
        c = (mix[:, 2 * mult:] * scale[2] + base[2 * mult:]).reshape(rows, mult, mult)
        c = torch.softmax(c, dim=2) + eps
        c = c / (c.sum(1, keepdim=True) + eps)
        for _ in range(1, iters):
            c = c / (c.sum(2, keepdim=True) + eps)
            c = c / (c.sum(1, keepdim=True) + eps)
        return pre, post, c
    _require(stream.is_contiguous() and fn.is_contiguous() and fn.dtype == BF16 and hidden % 8 == 0, "mhc mixes: layout")
    pre = torch.empty(rows, mult, dtype=torch.float32, device=stream.device)
    post = torch.empty_like(pre)
    comb = torch.empty(rows, mult, mult, dtype=torch.float32, device=stream.device)
    rc = kernels().ff_mhc_mixes(ptr(stream), ptr(fn), ptr(base), ptr(scale), rows, mult, hidden, iters, c_float(eps),
                                c_float(norm_eps), ptr(pre), ptr(post), ptr(comb), stream_ptr())
    check(rc, "ff_mhc_mixes")
    _count()
    return pre, post, comb


def collapse(stream: torch.Tensor, pre: torch.Tensor) -> torch.Tensor:
    rows, mult, hidden = stream.shape
    if not stream.is_cuda:
        acc = torch.zeros(rows, hidden)
        for j in range(mult):
            acc = acc + pre[:, j: j + 1] * stream[:, j].float()
        return acc.to(BF16)
    out = torch.empty(rows, hidden, dtype=BF16, device=stream.device)
    check(kernels().ff_mhc_collapse(ptr(stream), ptr(pre), rows, mult, hidden, ptr(out), stream_ptr()), "ff_mhc_collapse")
    _count()
    return out


def update(sub: torch.Tensor, residual: torch.Tensor, post: torch.Tensor, comb: torch.Tensor, rounding: int = 0,
           orientation: int = 0) -> torch.Tensor:
    rows, mult, hidden = residual.shape
    if not sub.is_cuda:
        c = comb if orientation == 0 else comb.transpose(1, 2)
        res = residual.float()
        if rounding == 1:
            p = post.to(BF16).float()
            prod = (p[:, :, None] * sub.float()[:, None, :]).to(BF16).float()
            mm = torch.einsum("rjk,rkh->rjh", c.to(BF16).float(), res).to(BF16).float()
            return (prod + mm).to(BF16)
        out = post[:, :, None] * sub.float()[:, None, :]
        for k in range(mult):
            out = out + c[:, :, k: k + 1] * res[:, k: k + 1, :]
        return out.to(BF16)
    out = torch.empty_like(residual)
    check(kernels().ff_mhc_update(ptr(sub), ptr(residual), ptr(post), ptr(comb), rows, mult, hidden, rounding, orientation,
                                  ptr(out), stream_ptr()), "ff_mhc_update")
    _count()
    return out
