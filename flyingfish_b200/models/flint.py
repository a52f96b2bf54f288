"""Flint-style decoder (the reference's ``Architecture::Flint``, src/model_spec.rs:2723-2905): every layer is GQA
attention with QK-norm and a *learnable soft-max* (one sink logit per query head that takes probability mass and carries
no value); most layers are local (sliding window, rotary positions), the listed ``no_rope_layers`` are global and use
no positional encoding at all. The first layers have a dense FFN, the rest sigmoid-routed experts with renormalised
top-k weights plus a shared expert.

Everything runs on the decoder's kernels: the sink is a denominator term of the prefill (tcgen05) and decode
attention kernels, the window is exact in both, a layer without positions writes its K/V through the rotary kernel
at position 0 (the identity rotation).
"""
from __future__ import annotations

import torch

from .. import ops
from .decoder import DecoderModel


class FlintModel(DecoderModel):
    def __init__(self, weights, comm=None, trace=None, seed: int = 0, state: dict[str, torch.Tensor] | None = None):
        super().__init__(weights, comm=comm, trace=trace)
        cfg = self.spec.extra["flint"]
        assert weights.tp.size == 1, "the Flint layout is served on one GPU per replica"
        assert self.d == 128 and self.spec.qk_norm, "128-wide heads with QK-norm"
        self.window = int(cfg["window"])
        self.no_rope = set(int(i) for i in cfg["no_rope_layers"])
        dev = weights.embed.device
        g = torch.Generator().manual_seed(seed + 313)
        self.sinks = []
        for i in range(self.spec.layers):
            if state is not None:
                sk = state[f"model.layers.{i}.self_attn.sinks"]
            else:
                sk = torch.randn(self.spec.heads, generator=g) * 1.5
            self.sinks.append(sk.float().contiguous().to(dev))
        self._zero_pos = None

    def is_global(self, i: int) -> bool:
        return i in self.no_rope

    def _attention(self, i, n, b, kv):
        lw, s = self.w.layers[i], self.spec
        glob = self.is_global(i)
        window = 0 if glob else self.window
        qkv = ops.linear(n, lw.wqkv)
        self._qk_norm(qkv, lw)
        if glob:
            # no positional encoding: the rotary kernel at position 0 is the identity and still writes K / V
            if self._zero_pos is None or self._zero_pos.numel() < b.positions.numel():
                self._zero_pos = torch.zeros(max(b.positions.numel(), 64), dtype=torch.int32, device=b.positions.device)
            pos = self._zero_pos[: b.positions.numel()]
        else:
            pos = b.positions
        ops.rope_kv_paged(qkv, pos, b.slots, kv.k[i], kv.v[i], self.hq, self.hkv, self.d, s.rope_theta)
        if b.is_decode:
            assert b.tree_mask is None, "tree verification is not available with a learnable soft-max"
            a = ops.attn_decode(qkv, kv.k[i], kv.v[i], b.block_table, b.ctx_lens, self.hq, self.hkv, self.d, self.scale,
                                nq=b.nq, max_ctx=b.max_ctx, window=window, sinks=self.sinks[i])
        else:
            a = ops.attn_prefill(qkv, kv.k[i], kv.v[i], b.block_table, b.q_start, b.q_lens, b.ctx_lens, b.max_q_len,
                                 self.hq, self.hkv, self.d, self.scale, window=window, sinks=self.sinks[i])
        if self.trace is not None:
            self.trace.record(f"layer.{i}.attn", a)
        return ops.linear(a, lw.wo)
