"""MoE operators: router, expert FFNs over routed rows, deterministic combine.

CPU tensors run the oracles in :mod:`flyingfish_b200.ops.ref`. CUDA tensors run the sm_100a
kernels of ``csrc/moe.cu``: one router kernel (logits + deterministic top-k for softmax /
sigmoid / grouped no-aux scoring), a device-side count/scan/permute that needs no host sync
(the reference reads the per-expert counts back to the host, src/backend/cuda/moe/prefill.rs:1137),
a grouped tcgen05 GEMM over the expert segments with SwiGLU in the epilogue, and a combine that
sums contributions in ascending expert id.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float

import torch

from . import ref
from .lib import check, kernels, ptr, status_tensor, stream_ptr


def route(x: torch.Tensor, w_router: torch.Tensor, top_k: int, score: str = "softmax",
          bias: torch.Tensor | None = None, n_groups: int = 1, topk_groups: int = 1, routed_scaling: float = 1.0,
          renormalize: bool = True) -> tuple[torch.Tensor, torch.Tensor]:
    """Returns (weights fp32 [rows, k], expert ids int32 [rows, k])."""
    if not x.is_cuda:
        return ref.moe_route(x, w_router, top_k, score, bias, n_groups, topk_groups, routed_scaling, renormalize)
    from . import moe_cuda
    return moe_cuda.route(x, w_router, top_k, score, bias, n_groups, topk_groups, routed_scaling, renormalize)


def experts_forward(x: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor, w_gate_up: torch.Tensor,
                    w_down: torch.Tensor, mode: int = 0) -> torch.Tensor:
    """Weighted sum of the selected experts' SwiGLU FFNs for every row (no shared expert)."""
    if not x.is_cuda:
        return ref.moe_forward(x, weights, ids, w_gate_up, w_down, None, None, mode)
    from . import moe_cuda
    return moe_cuda.experts_forward(x, weights, ids, w_gate_up, w_down, mode)


def add_shared(routed: torch.Tensor, shared: torch.Tensor) -> torch.Tensor:
    """Adds the shared expert's output in the storage dtype (one rounding)."""
    if not routed.is_cuda:
        return (routed.to(torch.float32) + shared.to(torch.float32)).to(routed.dtype)
    from . import residual_add
    return residual_add(routed, shared)
