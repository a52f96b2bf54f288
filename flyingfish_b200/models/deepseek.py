"""DeepSeek-V3-style decoder: multi-head latent attention (MLA) + dense / MoE feed-forward.

Attention runs in the absorbed form for prefill and decode alike: the cache holds one latent row
per token (``kv_lora_rank`` compressed KV + the shared RoPE key), queries are projected into the
latent space with W_UK, attention is multi-query over the latent rows, and the latent output is
expanded with W_UV before ``o_proj``. The FFN side (first dense layers, then grouped no-aux routed
experts + shared expert) reuses the decoder's MoE block. Reference for the operator sequence:
src/backend/cuda/engine_deepseek.rs:1119-1700 (latent mixer) and kernels/moe_route.cu:316-390.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from .. import ops
from ..config import ModelSpec
from ..ops import mla_ops
from .decoder import DecoderModel
from .weights import LayerWeights, ModelWeights, TPInfo, build_decoder_weights


@dataclass
class MlaWeights:
    q_a: torch.Tensor | None        # [q_lora, h]
    q_a_ln: torch.Tensor | None
    q_b: torch.Tensor               # [heads*(nope+rope), q_lora or h]
    kv_a: torch.Tensor              # [kv_lora + rope, h]
    kv_a_ln: torch.Tensor
    w_uk_t: torch.Tensor            # [heads, kv_lora, nope]   (absorb: q_lat = q_nope @ W_UK)
    w_uv: torch.Tensor              # [heads, v, kv_lora]
    wo: torch.Tensor                # [h, heads*v]


def build_deepseek_weights(spec: ModelSpec, source, device, tp: TPInfo | None = None, ep: TPInfo | None = None
                           ) -> ModelWeights:
    """FFN / norms / embeddings come from the common builder (with a stub attention geometry);
    the MLA projections are attached per layer as ``lw.extra['mla']``."""
    a = spec.mla
    heads = spec.heads

    # build with attention disabled: temporarily a spec whose attention tensors are tiny
    import copy
    stub = copy.copy(spec)
    stub.heads, stub.kv_heads, stub.head_dim = 1, 1, 16
    stub.qk_norm = False
    fp8 = spec.linear_format == "fp8_block"
    fp8_experts = spec.moe is not None and spec.moe.expert_format == "fp8_block"
    if fp8 != fp8_experts and spec.moe is not None:
        raise ValueError("FP8 DeepSeek-style checkpoints quantise the linears and the experts together")
    from .weights import pack_ffn_fp8
    w = build_decoder_weights(stub, source_with_stub_attention(source, device), device, tp, ep, fuse_swiglu=not fp8,
                              layer_hook=pack_ffn_fp8 if fp8 else None)
    w.spec = spec
    h = spec.hidden
    qk = a.qk_nope_dim + a.qk_rope_dim
    for i, lw in enumerate(w.layers):
        p = f"model.layers.{i}.self_attn."
        lw.wqkv = None
        if a.q_lora_rank:
            q_a = source(p + "q_a_proj.weight", (a.q_lora_rank, h))
            q_a_ln = source(p + "q_a_layernorm.weight", (a.q_lora_rank,))
            q_b = source(p + "q_b_proj.weight", (heads * qk, a.q_lora_rank))
        else:
            q_a, q_a_ln = None, None
            q_b = source(p + "q_proj.weight", (heads * qk, h))
        kv_a = source(p + "kv_a_proj_with_mqa.weight", (a.kv_lora_rank + a.qk_rope_dim, h))
        kv_a_ln = source(p + "kv_a_layernorm.weight", (a.kv_lora_rank,))
        kv_b = source(p + "kv_b_proj.weight", (heads * (a.qk_nope_dim + a.v_head_dim), a.kv_lora_rank))
        kv_b = kv_b.view(heads, a.qk_nope_dim + a.v_head_dim, a.kv_lora_rank)
        w_uk = kv_b[:, : a.qk_nope_dim]                         # [heads, nope, kv_lora]
        w_uv = kv_b[:, a.qk_nope_dim:].contiguous()             # [heads, v, kv_lora]
        wo = source(p + "o_proj.weight", (h, heads * a.v_head_dim))
        w_uk_t = w_uk.transpose(1, 2).contiguous()
        if fp8:
            # the projections stay in the checkpoint's E4M3 block format; the two absorbed factors of kv_b are small
            # and are applied per head in BF16
            from ..ops.quant_ops import Fp8Weight
            q_a = Fp8Weight.from_dense(q_a) if q_a is not None else None
            q_b, kv_a, wo = Fp8Weight.from_dense(q_b), Fp8Weight.from_dense(kv_a), Fp8Weight.from_dense(wo)
        lw.extra["mla"] = MlaWeights(q_a, q_a_ln, q_b, kv_a, kv_a_ln, w_uk_t, w_uv, wo)
        lw.wo = wo
    return w


def source_with_stub_attention(source, device):
    def src(name: str, shape):
        if any(k in name for k in (".self_attn.q_proj", ".self_attn.k_proj", ".self_attn.v_proj", ".self_attn.o_proj")):
            return torch.zeros(shape, dtype=torch.bfloat16, device=device)
        return source(name, shape)
    return src


class DeepseekModel(DecoderModel):
    """Same driver loop as :class:`DecoderModel`; only the attention block differs."""

    def __init__(self, weights: ModelWeights, comm=None, trace=None):
        super().__init__(weights, comm, trace)
        a = self.spec.mla
        self.mla = a
        self.scale = 1.0 / math.sqrt(a.qk_nope_dim + a.qk_rope_dim)
        self.latent_dim = a.kv_lora_rank + a.qk_rope_dim

    def _attention(self, i: int, n: torch.Tensor, b, kv) -> torch.Tensor:
        lw, s, a = self.w.layers[i], self.spec, self.mla
        m: MlaWeights = lw.extra["mla"]
        rows = n.shape[0]
        heads = s.heads
        if m.q_a is not None:
            qa = ops.rmsnorm(ops.linear(n, m.q_a), m.q_a_ln, s.rms_eps)
            q = ops.linear(qa, m.q_b)
        else:
            q = ops.linear(n, m.q_b)
        q = q.view(rows, heads, a.qk_nope_dim + a.qk_rope_dim)
        kva = ops.linear(n, m.kv_a)
        c = ops.rmsnorm(kva[:, : a.kv_lora_rank], m.kv_a_ln, s.rms_eps)
        k_rope = kva[:, a.kv_lora_rank:].contiguous()
        q_rope = q[:, :, a.qk_nope_dim:].reshape(rows, heads * a.qk_rope_dim).contiguous()
        ops.rope_inplace(q_rope, b.positions, heads, a.qk_rope_dim, s.rope_theta)
        ops.rope_inplace(k_rope, b.positions, 1, a.qk_rope_dim, s.rope_theta)
        mla_ops.cache_write(c, k_rope, b.slots, kv.k[i])
        q_lat = mla_ops.per_head_linear(q[:, :, : a.qk_nope_dim].contiguous(), m.w_uk_t)      # [rows, heads, kv_lora]
        q_full = torch.cat([q_lat, q_rope.view(rows, heads, a.qk_rope_dim)], dim=2).contiguous()
        if b.is_decode:
            batch = b.batch
            q_start = b.q_start
            q_lens = b.q_lens
            max_q = b.nq
        else:
            q_start, q_lens, max_q = b.q_start, b.q_lens, b.max_q_len
        out_lat = mla_ops.attention(q_full, kv.k[i], b.block_table, q_start, q_lens, b.ctx_lens, max_q,
                                    b.max_ctx, self.scale, a.kv_lora_rank)
        o = mla_ops.per_head_linear(out_lat, m.w_uv)                                          # [rows, heads, v]
        if self.trace is not None:
            self.trace.record(f"layer.{i}.attn", o)
        return self.comm.row_linear(o.reshape(rows, heads * a.v_head_dim), m.wo)
