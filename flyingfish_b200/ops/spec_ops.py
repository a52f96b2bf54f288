"""Speculative-decoding operators (``csrc/spec.cu``): the input rows of a multi-token-prediction module and greedy
chain acceptance on the device. CPU tensors run the oracles (the norm oracle of :mod:`ops.ref`, ``spec.accept``)."""
from __future__ import annotations

from ctypes import c_float

import torch

from . import _count, _require, ref
from .lib import check, kernels, ptr, status_tensor, stream_ptr


def mtp_mix(ids: torch.Tensor, table: torch.Tensor, hidden: torch.Tensor, enorm: torch.Tensor, hnorm: torch.Tensor,
            eps: float) -> torch.Tensor:
    """``[rmsnorm(embed[ids]) * enorm | rmsnorm(hidden) * hnorm]`` as one [rows, 2 * hidden] tensor."""
    if not table.is_cuda:
        e = ref.rmsnorm(table[ids.long()], enorm, eps, False)
        h = ref.rmsnorm(hidden, hnorm, eps, False)
        return torch.cat([e, h], dim=1).contiguous()
    rows, hdim = hidden.shape
    _require(ids.dtype == torch.int32 and ids.numel() == rows and hidden.stride(1) == 1, "mtp_mix: int32 ids, one per row")
    out = torch.empty(rows, 2 * hdim, dtype=torch.bfloat16, device=table.device)
    rc = kernels().ff_mtp_mix(ptr(ids), ptr(table), ptr(hidden), ptr(enorm), ptr(hnorm), ptr(out), rows, hdim,
                              table.shape[0], hidden.stride(0), c_float(eps), ptr(status_tensor(table.device)), stream_ptr())
    check(rc, "ff_mtp_mix")
    _count()
    return out


def accept_chain(draft: torch.Tensor, target: torch.Tensor, eos_ids: tuple[int, ...] = (), ignore_eos: bool = True
                 ) -> torch.Tensor:
    """``draft`` int32 [batch, k], ``target`` int32 [batch, k + 1] -> int32 [batch, k + 4] rows
    ``[accepted drafts, emitted tokens, hit_eos, tokens ... (-1 padded)]``."""
    batch, k = draft.shape
    if not draft.is_cuda:
        from ..spec.accept import accept_chain as host_accept
        out = torch.full((batch, k + 4), -1, dtype=torch.int32)
        for b in range(batch):
            a = host_accept(draft[b].tolist(), target[b].tolist(), eos_ids, ignore_eos)
            out[b, 0], out[b, 1], out[b, 2] = a.n_draft_accepted, len(a.tokens), int(a.hit_eos)
            out[b, 3: 3 + len(a.tokens)] = torch.tensor(a.tokens, dtype=torch.int32)
        return out
    _require(draft.dtype == torch.int32 and target.dtype == torch.int32 and target.shape == (batch, k + 1)
             and draft.is_contiguous() and target.is_contiguous(), "accept_chain: int32 [batch, k] / [batch, k + 1]")
    eos = torch.tensor(list(eos_ids) or [0], dtype=torch.int32, device=draft.device)
    out = torch.empty(batch, k + 4, dtype=torch.int32, device=draft.device)
    rc = kernels().ff_accept_chain(ptr(draft), ptr(target), ptr(eos), len(eos_ids), int(ignore_eos), batch, k, ptr(out),
                                   stream_ptr())
    check(rc, "ff_accept_chain")
    _count()
    return out
