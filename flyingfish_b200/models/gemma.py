"""Gemma-family decoder (Gemma-3 layout; the reference lists Gemma4 / EmbeddingGemma2 in src/model_spec.rs:8-104):
embeddings scaled by sqrt(hidden), RMSNorm weights stored as (w - 1), sandwich norms (a norm after the attention
and after the FFN output, before each residual add), QK-norm, tanh-GELU gated FFN, local layers with a sliding
window and their own rotary base interleaved with global layers (every ``global_every``-th), final logit soft-cap.

Everything runs on the decoder's kernels: the window is exact in prefill and decode attention (per-row visibility
sets), the extra norms are ``rmsnorm`` calls, the GeGLU is activation mode 2 of the SwiGLU kernels. Head width
stays 128 (the attention kernels' width); checkpoints with 256-wide heads are refused at load.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from .decoder import DecoderModel


class GemmaModel(DecoderModel):
    def __init__(self, weights, comm=None, trace=None, seed: int = 0, state: dict[str, torch.Tensor] | None = None):
        super().__init__(weights, comm=comm, trace=trace)
        cfg = self.spec.extra["gemma"]
        assert weights.tp.size == 1, "the Gemma layout is served on one GPU per replica"
        assert self.d == 128, "attention kernels are 128 wide"
        self.window = int(cfg.get("window", 512))
        self.global_every = int(cfg.get("global_every", 6))
        self.local_theta = float(cfg.get("local_rope_theta", 1e4))
        self.final_softcap = float(cfg.get("final_softcap", 0.0))
        self.embed_scale = float(cfg.get("embed_scale", math.sqrt(self.spec.hidden)))
        dev, dt = weights.embed.device, weights.embed.dtype
        g = torch.Generator().manual_seed(seed + 909)
        for i, lw in enumerate(weights.layers):
            for name, key in (("post_attn_ln", "post_attention_layernorm"), ("post_ffn_ln", "post_feedforward_layernorm")):
                if state is not None:
                    w = state[f"model.layers.{i}.{key}.weight"]
                else:
                    w = torch.randn(self.spec.hidden, generator=g) * 0.05          # stored as (w - 1)
                lw.extra[name] = w.to(dt).contiguous().to(dev)

    def is_global(self, i: int) -> bool:
        return (i + 1) % self.global_every == 0

    def _attention(self, i, n, b, kv):
        lw, s = self.w.layers[i], self.spec
        glob = self.is_global(i)
        theta = s.rope_theta if glob else self.local_theta
        window = 0 if glob else self.window
        qkv = ops.linear(n, lw.wqkv)
        rows = qkv.shape[0]
        q = qkv[:, : self.hq * self.d].reshape(rows * self.hq, self.d)
        k = qkv[:, self.hq * self.d: (self.hq + self.hkv) * self.d].reshape(rows * self.hkv, self.d)
        qkv[:, : self.hq * self.d] = ops.rmsnorm(q.contiguous(), lw.q_norm, s.rms_eps, unit_offset=True).view(rows, -1)
        qkv[:, self.hq * self.d: (self.hq + self.hkv) * self.d] = \
            ops.rmsnorm(k.contiguous(), lw.k_norm, s.rms_eps, unit_offset=True).view(rows, -1)
        ops.rope_kv_paged(qkv, b.positions, b.slots, kv.k[i], kv.v[i], self.hq, self.hkv, self.d, theta)
        if b.is_decode:
            a = ops.attn_decode(qkv, kv.k[i], kv.v[i], b.block_table, b.ctx_lens, self.hq, self.hkv, self.d, self.scale,
                                nq=b.nq, tree_mask=b.tree_mask if window == 0 else None, max_ctx=b.max_ctx, window=window)
        else:
            a = ops.attn_prefill(qkv, kv.k[i], kv.v[i], b.block_table, b.q_start, b.q_lens, b.ctx_lens, b.max_q_len,
                                 self.hq, self.hkv, self.d, self.scale, window=window)
        if self.trace is not None:
            self.trace.record(f"layer.{i}.attn", a)
        return ops.linear(a, lw.wo)

    def hidden_states(self, b, kv, inputs_embeds=None):
        w, s = self.w, self.spec
        x = ops.embed(b.ids, w.embed, scale=self.embed_scale) if inputs_embeds is None else inputs_embeds.clone()
        n = ops.rmsnorm(x, w.layers[0].input_ln, s.rms_eps, unit_offset=True)
        for i in range(s.layers):
            lw = w.layers[i]
            o = ops.rmsnorm(self._attention(i, n, b, kv), lw.extra["post_attn_ln"], s.rms_eps, unit_offset=True)
            n = ops.add_rmsnorm(o, x, lw.post_ln, s.rms_eps, unit_offset=True)          # x += o; pre-FFN norm
            f = ops.rmsnorm(self._ffn(i, n), lw.extra["post_ffn_ln"], s.rms_eps, unit_offset=True)
            next_w = w.layers[i + 1].input_ln if i + 1 < s.layers else w.final_norm
            n = ops.add_rmsnorm(f, x, next_w, s.rms_eps, unit_offset=True)
            if self.trace is not None:
                self.trace.record(f"layer.{i}", x)
        self.last_residual = x
        if self.normed_sink is not None:
            self.normed_sink.append(n)
        return n

    def logits(self, n, b):
        lg = super().logits(n, b)
        if self.final_softcap > 0:
            lg = ops.softcap(lg.contiguous(), self.final_softcap)
        return lg
