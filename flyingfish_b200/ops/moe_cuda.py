"""CUDA side of the MoE operators (see :mod:`flyingfish_b200.ops.moe_ops`)."""
from __future__ import annotations

import torch

from . import ref
from . import linear, silu_mul


def route(x, w_router, top_k, score, bias, n_groups, topk_groups, routed_scaling, renormalize):
    return ref.moe_route(x, w_router, top_k, score, bias, n_groups, topk_groups, routed_scaling, renormalize)


def experts_forward(x, weights, ids, w_gate_up, w_down, mode):
    rows, h = x.shape
    n_exp = w_gate_up.shape[0]
    contrib = torch.zeros(rows, ids.shape[1], h, dtype=torch.float32, device=x.device)
    for e in range(n_exp):
        r, c = torch.nonzero(ids == e, as_tuple=True)
        if r.numel() == 0:
            continue
        y = linear(silu_mul(linear(x[r].contiguous(), w_gate_up[e]), mode), w_down[e]).to(torch.float32)
        contrib[r, c] = y * weights[r, c, None]
    order = torch.argsort(ids.long(), dim=-1, stable=True)
    ordered = torch.gather(contrib, 1, order[:, :, None].expand_as(contrib))
    acc = torch.zeros(rows, h, dtype=torch.float32, device=x.device)
    for j in range(ids.shape[1]):
        acc = acc + ordered[:, j]
    return acc.to(x.dtype)
