"""Mixture-of-experts feed-forward block at model level.

Routing -> expert FFNs -> deterministic combine (+ shared expert). The semantics follow the
reference's MoE row oracle (src/backend/cuda/moe/reference.rs:332-605): top-k with ties to the
lower expert id, FP32 renormalised weights, contributions summed in ascending expert id and
rounded once, shared expert added afterwards. With expert parallelism the ``ep`` communicator of
the model dispatches token rows to the ranks that own the selected experts and combines their
outputs (see :mod:`flyingfish_b200.parallel.ep`).
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import moe_ops


def moe_cuda_mod():
    from ..ops import moe_cuda
    return moe_cuda


def moe_ffn(model, layer: int, n: torch.Tensor) -> torch.Tensor:
    lw = model.w.layers[layer]
    moe = model.spec.moe
    weights, ids = moe_ops.route(n, lw.router, moe.top_k, moe.score, lw.router_bias, moe.n_groups, moe.topk_groups,
                                 moe.routed_scaling, moe.renormalize)
    if getattr(model, "route_hook", None) is not None:
        model.route_hook(layer, ids, weights)
    ep = getattr(model, "ep", None)
    if ep is not None and ep.size > 1:
        routed = ep.dispatch_ffn_combine(n, weights, ids, lw, model.spec.swiglu_mode, layer=layer)
    else:
        provider = getattr(model, "expert_provider", None)
        fp4 = lw.extra.get("experts_fp4")
        if provider is not None:
            routed = provider.forward(layer, n, weights, ids)
        elif not isinstance(lw.experts_gu, torch.Tensor):
            # FP8-resident experts: grouped W8A8 GEMMs over the dispatched rows
            from ..ops import quant_ops
            routed = quant_ops.experts_forward_fp8(n, weights, ids, lw.experts_gu, lw.experts_down)
        elif (fp4 is not None and n.is_cuda
              and n.shape[0] * moe.top_k <= moe_cuda_mod().FP4_DECODE_MAX_ROWS * fp4[0].experts):
            # decode-sized call: packed NVFP4 experts expanded inside the grouped GEMM (a quarter of the bytes)
            routed = moe_cuda_mod().experts_forward_nvfp4(n, weights, ids, fp4[0], fp4[1])
        else:
            routed = moe_ops.experts_forward(n, weights, ids, lw.experts_gu, lw.experts_down, model.spec.swiglu_mode)
    if lw.shared_gu is not None:
        sh = ops.silu_mul(ops.linear(n, lw.shared_gu), mode=model.spec.swiglu_mode)
        shared = model.comm.row_linear(sh, lw.shared_down)
        routed = moe_ops.add_shared(routed, shared)
    return routed
