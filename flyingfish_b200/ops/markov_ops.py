"""Markov head of the tree drafter (DSpark): per request, ``s = bf16(bf16(w2 @ w1[parent]) + base_logits)``, its
top-4 tokens (ties to the smaller id), their log-probabilities and the log-sum-exp. CUDA: the decode GEMM for the
bias and ``csrc/markov.cu`` for the row-wise top-4 / log-sum-exp; CPU: oracle (reference: kernels/markov.cu:1-55)."""
from __future__ import annotations

import torch

from . import _count, linear, workspace
from .lib import check, kernels, ptr, stream_ptr

BF16 = torch.bfloat16


def markov_top4(w1: torch.Tensor, w2: torch.Tensor, base: torch.Tensor, req_tok: torch.Tensor, req_row: torch.Tensor
                ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """w1, w2 [V, 256] bf16, base [rows, V] bf16 logits, req_tok / req_row [P] -> top4 [P, 4] int32,
    logp [P, 4] f32, lse [P] f32."""
    p_, v = req_tok.numel(), w2.shape[0]
    parent = w1[req_tok.long()]                                     # [P, 256]
    bias = linear(parent, w2)                                       # [P, V] bf16 (the first rounding point)
    if not base.is_cuda:
        s = (bias.float() + base[req_row.long()].float()).to(BF16).float()
        top4 = torch.empty(p_, 4, dtype=torch.int32); logp = torch.empty(p_, 4); lse = torch.empty(p_)
        for i in range(p_):
            order = sorted(range(v), key=lambda j: (-float(s[i, j]), j))[:4]
            m = s[i].max()
            logsum = torch.log(torch.exp(s[i] - m).sum())
            top4[i] = torch.tensor(order, dtype=torch.int32)
            logp[i] = (s[i, order] - m) - logsum
            lse[i] = m + logsum
        return top4, logp, lse
    chunks = (v + 4095) // 4096
    ws = workspace(base.device)
    part_top = ws.ensure("markov_top", p_ * chunks * 8)
    part_ml = ws.ensure("markov_ml", p_ * chunks * 2)
    top4 = torch.empty(p_, 4, dtype=torch.int32, device=base.device)
    logp = torch.empty(p_, 4, dtype=torch.float32, device=base.device)
    lse = torch.empty(p_, dtype=torch.float32, device=base.device)
    rc = kernels().ff_markov_top4(ptr(bias), ptr(base), ptr(req_row), p_, v, bias.stride(0), base.stride(0), ptr(part_top),
                                  ptr(part_ml), ptr(top4), ptr(logp), ptr(lse), stream_ptr())
    check(rc, "ff_markov_top4")
    _count(2)
    return top4, logp, lse
