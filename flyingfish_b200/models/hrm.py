"""Looped two-stack decoder (the text model of the reference's ``Architecture::LoopVl``, ``HrmTextForCausalLM``:
src/model_spec.rs:2290-2400, src/backend/cuda/engine_recurrent.rs:1004-1300).

Two token-aligned states, ``high`` (the scaled embeddings) and ``low`` (a learned initial vector), are refined by two
weight stacks: every H cycle runs the L stack ``l_cycles`` times on ``low`` (input ``low + high``) and then the H stack
once on ``high`` (input ``high + low``). A stack call is a run of pre-norm layers with weight-less RMSNorm, gated
attention (``o_proj(attn * sigmoid(gate))``, the gate being a fourth slice of the fused projection) and a SwiGLU FFN; the
call's result is the norm of its last residual. Every layer *application* has its own KV cache layer, so the model has
``h_cycles * (l_cycles + 1) * layers_per_stack`` cache layers over ``2 * layers_per_stack`` weight sets. Positions use
YaRN-scaled rotary tables whose attention factor is folded into cos / sin. The prompt is encoded bidirectionally (every
prompt token sees the whole prompt), generated tokens attend causally; the logits come from ``high`` without a final
norm.

The image side of LoopVL (vision encoder, projector, visual re-injection gate) is not part of this module.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..config import ModelSpec
from ..ops import vision_ops
from .decoder import DecoderModel
from .weights import DTYPES, LayerWeights, ModelWeights, TPInfo, TensorSource, synthetic_source


def yarn_inv_freq(dim: int, theta: float, factor: float, original_max: int, beta_fast: float, beta_slow: float) -> torch.Tensor:
    """[dim / 2] inverse frequencies: interpolated (divided by ``factor``) below the ``beta_slow`` rotation count,
    untouched above ``beta_fast``, a linear ramp between; values rounded to BF16."""
    def correction(rotations: float) -> float:
        return dim * math.log(original_max / (rotations * 2.0 * math.pi)) / (2.0 * math.log(theta))
    low = max(math.floor(correction(beta_fast)), 0.0)
    high = min(math.ceil(correction(beta_slow)), dim - 1.0)
    d = torch.arange(dim // 2, dtype=torch.float32)
    extrapolation = 1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32), 2.0 * d / dim)
    ramp = ((d - low) / max(high - low, 1e-3)).clamp(0.0, 1.0)
    inv = extrapolation / factor * ramp + extrapolation * (1.0 - ramp)
    return inv.to(torch.bfloat16).float()


def build_hrm_weights(spec: ModelSpec, source: TensorSource, device: torch.device) -> ModelWeights:
    """Weight sets of the L stack then the H stack (checkpoint names ``language_model.model.{L,H}_module.layers.N``);
    Q, K, V and the gate projection are fused into one [4 * hidden, hidden] matrix."""
    cfg = spec.extra["hrm"]
    h, f, per = spec.hidden, spec.ffn, int(cfg["layers_per_stack"])
    layers = []
    for stack in ("L", "H"):
        for i in range(per):
            p = f"language_model.model.{stack}_module.layers.{i}"
            fused = torch.cat([source(f"{p}.self_attn.{r}_proj.weight", (h, h)) for r in ("q", "k", "v", "gate")], dim=0)
            gu = torch.cat([source(f"{p}.mlp.gate_proj.weight", (f, h)), source(f"{p}.mlp.up_proj.weight", (f, h))], dim=0)
            layers.append(LayerWeights(wqkv=fused.contiguous(), wo=source(f"{p}.self_attn.o_proj.weight", (h, h)),
                                       wgu=gu.contiguous(), wgu_interleaved=False, wdown=source(f"{p}.mlp.down_proj.weight", (h, f))))
    embed = source("language_model.model.embed_tokens.weight", (spec.vocab, h))
    head = source("language_model.lm_head.weight", (spec.vocab, h))
    z_l = source("language_model.model.z_L_init", (h,))
    ones = torch.ones(h, dtype=embed.dtype, device=device)
    return ModelWeights(spec=spec, embed=embed, final_norm=ones, lm_head=head, layers=layers, tp=TPInfo(),
                        vocab_shard=(0, spec.vocab), extra={"z_l_init": z_l})


def random_hrm_weights(spec: ModelSpec, seed: int, device: torch.device | str) -> ModelWeights:
    device = torch.device(device)
    dtype = DTYPES[spec.dtype] if device.type == "cuda" else torch.float32
    return build_hrm_weights(spec, synthetic_source(spec, seed, device, dtype), device)


class HrmModel(DecoderModel):
    whole_prompt_prefill = True        # the prompt is encoded bidirectionally: the engine never splits one over chunks

    def __init__(self, weights: ModelWeights, comm=None, trace=None):
        super().__init__(weights, comm=comm, trace=trace)
        cfg = self.spec.extra["hrm"]
        assert weights.tp.size == 1, "the looped model is served on one GPU per replica"
        assert self.hq == self.hkv and self.d == 128, "full multi-head attention with 128-wide heads"
        self.per = int(cfg["layers_per_stack"])
        self.h_cycles, self.l_cycles = int(cfg["h_cycles"]), int(cfg["l_cycles"])
        self.embedding_scale = float(cfg["embedding_scale"])
        y = cfg["yarn"]
        dev = weights.embed.device
        self.inv_freq = yarn_inv_freq(self.d, self.spec.rope_theta, y["factor"], y["original_max"], y["beta_fast"], y["beta_slow"]).to(dev)
        self.rope_scale = 0.1 * math.log(y["factor"]) + 1.0
        # (high stack?, first cache layer) of every stack call, in execution order
        calls = self.h_cycles * (self.l_cycles + 1)
        self.program = [((c % (self.l_cycles + 1)) == self.l_cycles, c * self.per) for c in range(calls)]
        assert self.spec.layers == calls * self.per, "spec.layers counts one cache layer per layer application"
        self.z_l = weights.extra["z_l_init"]
        self.ones = weights.final_norm

    def _rope_table(self, positions: torch.Tensor) -> torch.Tensor:
        ang = positions.to(torch.float32)[:, None] * self.inv_freq[None, :]
        cs = (torch.cos(ang) * self.rope_scale).to(torch.bfloat16).float()
        sn = (torch.sin(ang) * self.rope_scale).to(torch.bfloat16).float()
        return torch.stack([cs, sn], dim=-1).contiguous()

    def _layer(self, lw: LayerWeights, slot: int, n, x, b, kv, table):
        s, h = self.spec, self.spec.hidden
        qkvg = ops.linear(n, lw.wqkv)
        vision_ops.rope_table_apply_(qkvg, table, self.hq, self.d, self.d, b.slots, kv.k[slot], kv.v[slot], self.hkv)
        if b.is_decode:
            a = ops.attn_decode(qkvg, kv.k[slot], kv.v[slot], b.block_table, b.ctx_lens, self.hq, self.hkv, self.d, self.scale,
                                nq=b.nq, tree_mask=b.tree_mask, max_ctx=b.max_ctx)
        else:
            a = ops.attn_prefill(qkvg, kv.k[slot], kv.v[slot], b.block_table, b.q_start, b.q_lens, b.ctx_lens, b.max_q_len,
                                 self.hq, self.hkv, self.d, self.scale, window=-1)
        g = vision_ops.sigmoid_gate(a, qkvg[:, 3 * h: 4 * h])
        n = ops.add_rmsnorm(ops.linear(g, lw.wo), x, self.ones, s.rms_eps)
        hmid = ops.silu_mul(ops.linear(n, lw.wgu), mode=s.swiglu_mode)
        return ops.add_rmsnorm(ops.linear(hmid, lw.wdown), x, self.ones, s.rms_eps)

    def hidden_states(self, b, kv, inputs_embeds: torch.Tensor | None = None) -> torch.Tensor:
        assert inputs_embeds is None, "the looped model takes token ids"
        w, s = self.w, self.spec
        table = self._rope_table(b.positions)
        high = ops.embed(b.ids, w.embed, self.embedding_scale)
        low = self.z_l.to(high.dtype)[None, :].expand(high.shape[0], -1).contiguous()
        for is_high, offset in self.program:
            target, other = (high, low) if is_high else (low, high)
            x = target.clone()
            n = ops.add_rmsnorm(other, x, self.ones, s.rms_eps)
            base = self.per if is_high else 0
            for layer in range(self.per):
                n = self._layer(w.layers[base + layer], offset + layer, n, x, b, kv, table)
            if is_high:
                high = n
            else:
                low = n
            if self.trace is not None:
                self.trace.record(f"stack.{offset // self.per}", n)
        self.last_residual = high
        if self.normed_sink is not None:
            self.normed_sink.append(high)
        return high
