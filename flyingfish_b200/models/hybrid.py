"""Hybrid decoder: gated-delta-net (linear attention) mixers in most layers, full attention in every
``full_attention_interval``-th one (the Qwen3.5-text / Qwen3-Next layout; reference: ``Mixer{FullAttention,Gdn}``
in src/model_spec.rs:8-104, kernels/gdn/*).

A gated-delta-net layer:
    proj        = x W_in^T                       columns: q | k (k_heads x 128 each) | v | z (v_heads x 128 each) | b | a
    q, k, v     = SiLU(causal depthwise conv4(q | k | v))           conv history carried per sequence
    q, k        = l2norm(q) / sqrt(128), l2norm(k)                  (k heads repeated over the value heads)
    beta, g     = sigmoid(b), -exp(A_log) * softplus(a + dt_bias)
    S           = S * exp(g);  delta = (v - S^T k) * beta;  S += k delta^T;  o = S^T q        per token, per head
    y           = (rmsnorm_128(o) * norm_w * SiLU(z)) W_out^T
Per-sequence state (conv history [conv_dim, 3], S [v_heads, 128, 128], both FP32) lives in slot-indexed slabs; the
engine hands every sequence a slot and names the slots of a batch in ``ForwardBatch.state_slots``. The step is
the same for prefill chunks and decode rows (the kernels walk each sequence's rows in order), so a chunked
prefill and token-by-token decoding produce the same state. Decode steps replay from CUDA graphs (slots and row
ranges are views of the packed step metadata). Not supported with this mixer: speculative rollback, tensor parallelism.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .. import ops
from ..ops import gdn_ops
from .decoder import DecoderModel

D = 128


@dataclass
class GdnWeights:
    w_in: torch.Tensor          # [2*kh*128 + 2*vh*128 + pad8(2*vh), hidden]
    conv_w: torch.Tensor        # [2*kh*128 + vh*128, 4]
    a_log: torch.Tensor         # [vh] f32
    dt_bias: torch.Tensor       # [vh] f32
    norm_w: torch.Tensor        # [128]
    w_out: torch.Tensor         # [hidden, vh*128]


class HybridModel(DecoderModel):
    def __init__(self, weights, comm=None, trace=None, max_sequences: int = 64, seed: int = 0,
                 state: dict[str, torch.Tensor] | None = None):
        super().__init__(weights, comm=comm, trace=trace)
        cfg = self.spec.extra["gdn"]
        assert weights.tp.size == 1, "gated-delta-net layers are not tensor-parallel"
        self.vh, self.kh = int(cfg["v_heads"]), int(cfg["k_heads"])
        interval = int(cfg.get("full_attention_interval", 4))
        self.gdn_layers = {i for i in range(self.spec.layers) if (i + 1) % interval != 0}
        self.conv_dim = (2 * self.kh + self.vh) * D
        self.value_dim = self.vh * D
        dev, dt = weights.embed.device, weights.embed.dtype
        g = torch.Generator().manual_seed(seed + 4242)
        hidden = self.spec.hidden
        n_in = self.conv_dim + self.value_dim + (2 * self.vh + 7) // 8 * 8
        self.gdn: dict[int, GdnWeights] = {}
        for i in sorted(self.gdn_layers):
            p = f"model.layers.{i}.linear_attn."
            if state is not None:
                t = lambda n: state[p + n]
                w_in, conv_w, a_log, dt_b, norm_w, w_out = (t("in_proj.weight"), t("conv1d.weight"), t("A_log"),
                                                            t("dt_bias"), t("norm.weight"), t("out_proj.weight"))
            else:
                w_in = torch.randn(n_in, hidden, generator=g) * 0.02
                conv_w = torch.randn(self.conv_dim, 4, generator=g) * 0.3
                a_log = torch.log(torch.rand(self.vh, generator=g) * 3 + 0.5)
                dt_b = torch.randn(self.vh, generator=g) * 0.5
                norm_w = torch.ones(D) + torch.randn(D, generator=g) * 0.02
                w_out = torch.randn(hidden, self.value_dim, generator=g) * 0.02
            self.gdn[i] = GdnWeights(w_in.to(dt).contiguous().to(dev), conv_w.to(torch.bfloat16).contiguous().to(dev),
                                     a_log.float().to(dev), dt_b.float().to(dev), norm_w.to(dt).contiguous().to(dev),
                                     w_out.to(dt).contiguous().to(dev))
        self.state_slot_count = max_sequences + 1
        self.conv_hist = {i: torch.zeros(self.state_slot_count, self.conv_dim, 3, dtype=torch.float32, device=dev)
                          for i in self.gdn_layers}
        self.rec_state = {i: torch.zeros(self.state_slot_count, self.vh, D, D, dtype=torch.float32, device=dev)
                          for i in self.gdn_layers}
        self._meta = None

    def reset_state(self, slot: int) -> None:
        for i in self.gdn_layers:
            self.conv_hist[i][slot].zero_()
            self.rec_state[i][slot].zero_()

    def state_bytes_per_sequence(self) -> int:
        return len(self.gdn_layers) * 4 * (self.conv_dim * 3 + self.vh * D * D)

    graph_safe_state = True          # slots and row ranges come from the packed step metadata (fixed device addresses)

    def hidden_states(self, b, kv, inputs_embeds=None):
        # row ranges and state slots of the sequences in this batch, shared by every gated-delta-net layer: views of
        # the packed metadata buffer, so a captured decode step sees each step's values
        if getattr(b, "layout", None) is not None and hasattr(b, "row_start"):
            assert getattr(b, "state_slots", None) is not None and len(b.state_slots) == b.batch, \
                "the engine must name a state slot per sequence of the batch"
            self._meta = (b.row_start, b.state_slots_dev)
        else:
            lens = b.q_lens.cpu().tolist() if not isinstance(b.q_lens, list) else b.q_lens
            starts, acc = [0], 0
            for n in lens:
                acc += int(n)
                starts.append(acc)
            slots = list(getattr(b, "state_slots", None) or [])
            assert len(slots) == len(lens), "the engine must name a state slot per sequence of the batch"
            dev = self.w.embed.device
            self._meta = (torch.tensor(starts, dtype=torch.int32, device=dev), torch.tensor(slots, dtype=torch.int32, device=dev))
        return super().hidden_states(b, kv, inputs_embeds)

    def _attention(self, i, n, b, kv):
        if i not in self.gdn_layers:
            return super()._attention(i, n, b, kv)
        g = self.gdn[i]
        row_start, slots = self._meta
        rows = n.shape[0]
        proj = ops.linear(n, g.w_in)
        if proj.dtype != torch.bfloat16:
            proj = proj.to(torch.bfloat16)
        conv_out = gdn_ops.conv_batched(proj, g.conv_w, self.conv_hist[i], row_start, slots)
        q, k, v = gdn_ops.prep(conv_out, self.vh, self.kh)
        z = proj[:, self.conv_dim: self.conv_dim + self.value_dim]
        ba = proj[:, self.conv_dim + self.value_dim: self.conv_dim + self.value_dim + 2 * self.vh].float()
        beta = torch.sigmoid(ba[:, : self.vh]).contiguous()
        dec = (-torch.exp(g.a_log)[None, :] * F.softplus(ba[:, self.vh:] + g.dt_bias[None, :])).contiguous()
        # prefill chunks go through the chunked (tensor-core) form of the recurrence, decode rows through the
        # token-by-token kernel
        step = gdn_ops.chunked_slots if (not b.is_decode and b.max_q_len >= gdn_ops.CHUNK_MIN_ROWS) else gdn_ops.recurrent_slots
        o = step(q, k, v, beta, dec, self.rec_state[i], row_start, slots)                         # [rows, vh, 128] bf16
        on = ops.rmsnorm(o.reshape(rows * self.vh, D).to(g.norm_w.dtype), g.norm_w, self.spec.rms_eps)
        y = (on.reshape(rows, self.value_dim).float() * F.silu(z.float())).to(g.w_out.dtype)
        if self.trace is not None:
            self.trace.record(f"layer.{i}.gdn", y)
        return self.comm.row_linear(y.contiguous(), g.w_out)
