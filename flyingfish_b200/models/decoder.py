"""GQA decoder (Llama / Qwen3 / tiny-MoE / Qwen3-MoE shapes) on the operator API.

Layer program (the reference's dense Llama program, src/backend/cuda/engine.rs:2776-3330):

    embed+rmsnorm -> per layer { QKV linear -> RoPE + paged KV write -> attention -> O linear
    -> add+rmsnorm -> gate/up linear (+SwiGLU in the epilogue) -> down linear -> add+rmsnorm }
    -> lm_head on the selected rows -> argmax

The residual stream and the normalised activations are separate buffers; with tensor
parallelism the row-parallel projections (O, down) end in an all-reduce supplied by the
``comm`` object (fused into the GEMM kernel when the symmetric-memory path is active), the
QKV / gate-up / lm_head projections are column-parallel and the final argmax merges
vocabulary shards.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from ..config import ModelSpec
from ..engine.batch import ForwardBatch
from ..engine.kv_cache import PagedKVCache
from .weights import ModelWeights
from . import moe as moe_mod


class NoComm:
    """Single-rank stand-in for the tensor-parallel communicator."""
    rank, size = 0, 1

    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def row_linear(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, w)

    def all_gather_cat(self, x: torch.Tensor) -> torch.Tensor:
        return x


class DecoderModel:
    def __init__(self, weights: ModelWeights, comm=None, trace=None):
        self.w = weights
        self.spec: ModelSpec = weights.spec
        self.comm = comm or NoComm()
        tp = weights.tp.size
        self.hq = self.spec.heads // tp
        self.hkv = max(1, self.spec.kv_heads // tp)
        self.d = self.spec.head_dim
        self.scale = 1.0 / math.sqrt(self.d)
        self.trace = trace           # optional flyingfish_b200.utils.trace.Trace
        self.capture_taps: dict[int, int] = {}    # layer index -> tap slot for draft-model hidden taps
        self.capture_slab: torch.Tensor | None = None
        self.normed_sink: list | None = None      # when a list: every forward appends its final-normed rows
        self._rope_cs: torch.Tensor | None = None  # per-forward cos/sin table of the fused QKV kernels
        # encoders and diffusion language models attend in both directions inside a sequence; they run whole
        # sequences in one prefill chunk and never decode
        self.bidirectional = bool(self.spec.extra.get("bidirectional"))

    # -- pieces ----------------------------------------------------------------------------
    def _attention(self, i: int, n: torch.Tensor, b: ForwardBatch, kv: PagedKVCache) -> torch.Tensor:
        lw, s = self.w.layers[i], self.spec
        if s.qk_norm:
            qkv = ops.linear(n, lw.wqkv)
            self._qk_norm(qkv, lw)
            ops.rope_kv_paged(qkv, b.positions, b.slots, kv.k[i], kv.v[i], self.hq, self.hkv, self.d, s.rope_theta)
        else:
            qkv = ops.linear_rope_kv(n, lw.wqkv, b.positions, b.slots, kv.k[i], kv.v[i], self.hq, self.hkv, self.d,
                                     s.rope_theta, cos_sin=self._rope_cs)
        if b.is_decode and kv.compact is not None and b.kv_start is not None:
            # older keys live in the sealed 8-bit store: BF16 pages + sealed groups, one merge
            a = ops.attn_decode_mixed(qkv, kv.k[i], kv.v[i], kv.compact, i, b.block_table, b.ctx_lens, b.kv_start,
                                      b.group_table, self.hq, self.hkv, self.d, self.scale, max_ctx=b.max_ctx)
        elif b.is_decode:
            a = ops.attn_decode(qkv, kv.k[i], kv.v[i], b.block_table, b.ctx_lens, self.hq, self.hkv, self.d,
                                self.scale, nq=b.nq, tree_mask=b.tree_mask, max_ctx=b.max_ctx)
        else:
            a = ops.attn_prefill(qkv, kv.k[i], kv.v[i], b.block_table, b.q_start, b.q_lens, b.ctx_lens, b.max_q_len,
                                 self.hq, self.hkv, self.d, self.scale, window=-1 if self.bidirectional else 0)
        if self.trace is not None:
            self.trace.record(f"layer.{i}.attn", a)
        return self.comm.row_linear(a, lw.wo)

    def _qk_norm(self, qkv: torch.Tensor, lw) -> None:
        rows = qkv.shape[0]
        q = qkv[:, : self.hq * self.d].reshape(rows * self.hq, self.d)
        k = qkv[:, self.hq * self.d: (self.hq + self.hkv) * self.d].reshape(rows * self.hkv, self.d)
        qn = ops.rmsnorm(q.contiguous(), lw.q_norm, self.spec.rms_eps)
        kn = ops.rmsnorm(k.contiguous(), lw.k_norm, self.spec.rms_eps)
        qkv[:, : self.hq * self.d] = qn.view(rows, -1)
        qkv[:, self.hq * self.d: (self.hq + self.hkv) * self.d] = kn.view(rows, -1)

    def _ffn(self, i: int, n: torch.Tensor) -> torch.Tensor:
        lw = self.w.layers[i]
        if lw.router is not None:
            return moe_mod.moe_ffn(self, i, n)
        if lw.wgu_interleaved:
            hmid = ops.linear_swiglu(n, lw.wgu, mode=self.spec.swiglu_mode)
        else:
            hmid = ops.silu_mul(ops.linear(n, lw.wgu), mode=self.spec.swiglu_mode)
        return self.comm.row_linear(hmid, lw.wdown)

    # -- forward ---------------------------------------------------------------------------
    def hidden_states(self, b: ForwardBatch, kv: PagedKVCache, inputs_embeds: torch.Tensor | None = None
                      ) -> torch.Tensor:
        """Runs all layers; returns the final-normed activations [rows, hidden]. ``inputs_embeds``
        replaces the embedding lookup (multi-token-prediction heads feed a projected mix of the
        next token's embedding and the previous hidden state)."""
        w, s = self.w, self.spec
        self._rope_cs = None
        if inputs_embeds is None and self._sequence_parallel(b):
            return self._hidden_states_sp(b, kv)
        if self._chain_ok(b):
            return self._hidden_states_chain(b, kv, inputs_embeds)
        if b.positions.is_cuda and b.positions.shape[0] <= ops.SKINNY_MAX_M and self.d == 128 and not s.qk_norm:
            # one cos/sin table per step for the fused QKV + rotary + KV-write kernels of all layers
            self._rope_cs = ops.rope_table(b.positions, self.d, s.rope_theta)
        if inputs_embeds is None:
            x, n = ops.embed_rmsnorm(b.ids, w.embed, w.layers[0].input_ln, s.rms_eps)
        else:
            x = inputs_embeds.clone()
            n = ops.rmsnorm(x, w.layers[0].input_ln, s.rms_eps)
        if self.trace is not None:
            self.trace.record("embed", x)
        for i in range(s.layers):
            lw = w.layers[i]
            o = self._attention(i, n, b, kv)
            n = ops.add_rmsnorm(o, x, lw.post_ln, s.rms_eps)
            dn = self._ffn(i, n)
            next_w = w.layers[i + 1].input_ln if i + 1 < s.layers else w.final_norm
            cap = None
            if i in self.capture_taps and self.capture_slab is not None:
                cap = self.capture_slab[: x.shape[0], self.capture_taps[i]]
            n = ops.add_rmsnorm(dn, x, next_w, s.rms_eps, capture=cap)
            if self.trace is not None:
                self.trace.record(f"layer.{i}", x)
        self.last_residual = x
        if self.normed_sink is not None:
            self.normed_sink.append(n)
        return n

    # -- decode through the per-layer projection chain ------------------------------------------
    def _chain_ok(self, b: ForwardBatch) -> bool:
        """Decode batches of a dense layer stack on one GPU run every layer's projections and norms as one
        persistent kernel (``ops/chain.py``); everything it does not cover takes the operator-by-operator path."""
        from ..ops import chain
        s = self.spec
        if not (chain.ENABLED and b.is_decode and b.positions.is_cuda and b.rows <= chain.MAX_ROWS):
            return False
        if getattr(b, "kv_start", None) is not None:
            return False
        if getattr(self.comm, "size", 1) != 1 or self.trace is not None or self.capture_taps or s.qk_norm:
            return False
        if self.d != 128 or s.hidden > chain.MAX_HIDDEN or s.hidden % 128 or s.swiglu_mode != 0:
            return False
        for lw in self.w.layers:
            if lw.router is not None or not lw.wgu_interleaved or lw.wgu.shape[0] % 256 or lw.wdown.shape[1] % 8:
                return False
        return True

    def _hidden_states_chain(self, b: ForwardBatch, kv: PagedKVCache, inputs_embeds: torch.Tensor | None) -> torch.Tensor:
        from ..ops import chain
        w, s = self.w, self.spec
        cs = ops.rope_table(b.positions, self.d, s.rope_theta)
        if inputs_embeds is None:
            x, n = ops.embed_rmsnorm(b.ids, w.embed, w.layers[0].input_ln, s.rms_eps)
        else:
            x = inputs_embeds.clone()
            n = ops.rmsnorm(x, w.layers[0].input_ln, s.rms_eps)
        qkv = ops.linear_rope_kv(n, w.layers[0].wqkv, b.positions, b.slots, kv.k[0], kv.v[0], self.hq, self.hkv, self.d,
                                 s.rope_theta, cos_sin=cs)
        for i in range(s.layers):
            lw = w.layers[i]
            a = ops.attn_decode(qkv, kv.k[i], kv.v[i], b.block_table, b.ctx_lens, self.hq, self.hkv, self.d, self.scale,
                                nq=b.nq, tree_mask=b.tree_mask, max_ctx=b.max_ctx)
            last = i + 1 == s.layers
            rope = None if last else {"cos_sin": cs, "slots": b.slots, "kcache": kv.k[i + 1], "vcache": kv.v[i + 1],
                                      "hq": self.hq, "hkv": self.hkv, "rot_dim": self.d}
            n, qkv = chain.layer_chain(a, x, lw.wo, lw.post_ln, lw.wgu, lw.wdown,
                                       w.final_norm if last else w.layers[i + 1].input_ln, s.rms_eps,
                                       None if last else w.layers[i + 1].wqkv, rope)
            ops._count()
        self.last_residual = x
        if self.normed_sink is not None:
            self.normed_sink.append(n)
        return n

    # -- sequence-parallel prefill (tensor parallel, fused AG->GEMM / GEMM->RS) -------------------
    def _sequence_parallel(self, b: ForwardBatch) -> bool:
        c = self.comm
        if getattr(c, "size", 1) < 2 or b.is_decode or not getattr(c, "fused", False) or self.trace is not None:
            return False
        if self.bidirectional:
            return False
        if any(lw.router is not None or not lw.wgu_interleaved for lw in self.w.layers) or self.spec.qk_norm:
            return False
        f_local = self.w.layers[0].wdown.shape[1]
        return c.sp_ok(b.rows, self.spec.hidden, self.spec.hidden) and (2 * f_local) % 256 == 0

    def _hidden_states_sp(self, b: ForwardBatch, kv: PagedKVCache) -> torch.Tensor:
        """Activations between the projections are row-sharded over the ranks (each owns
        ``rows / world`` rows of the residual stream); QKV and gate/up run as all-gather -> GEMM,
        O and down as GEMM -> reduce-scatter, each one fused kernel."""
        w, s, c = self.w, self.spec, self.comm
        rpr = b.rows // c.size
        r0 = c.rank * rpr
        x, n = ops.embed_rmsnorm(b.ids[r0: r0 + rpr].contiguous(), w.embed, w.layers[0].input_ln, s.rms_eps)
        for i in range(s.layers):
            lw = w.layers[i]
            qkv = c.ag_linear(n, lw.wqkv)
            ops.rope_kv_paged(qkv, b.positions, b.slots, kv.k[i], kv.v[i], self.hq, self.hkv, self.d, s.rope_theta)
            a = torch.zeros(b.rows, self.hq * self.d, dtype=qkv.dtype, device=qkv.device)    # padding rows stay finite
            ops.attn_prefill(qkv, kv.k[i], kv.v[i], b.block_table, b.q_start, b.q_lens, b.ctx_lens, b.max_q_len,
                             self.hq, self.hkv, self.d, self.scale, out=a)
            o = c.rs_linear(a, lw.wo)
            n = ops.add_rmsnorm(o, x, lw.post_ln, s.rms_eps)
            hmid = c.ag_linear(n, lw.wgu, swiglu=True)
            dn = c.rs_linear(hmid, lw.wdown)
            next_w = w.layers[i + 1].input_ln if i + 1 < s.layers else w.final_norm
            n = ops.add_rmsnorm(dn, x, next_w, s.rms_eps)
        full = c.all_gather_rows(n)
        if self.normed_sink is not None:
            self.normed_sink.append(full)
        return full

    def logits(self, n: torch.Tensor, b: ForwardBatch) -> torch.Tensor:
        """lm_head on the rows named by ``b.logit_rows`` -> [n_rows, local vocab]."""
        sel = n.index_select(0, b.logit_rows.long()) if b.n_logit_rows != n.shape[0] else n
        return ops.linear(sel.contiguous(), self.w.lm_head)

    def greedy(self, logits: torch.Tensor) -> torch.Tensor:
        tp = self.w.tp
        if tp.size == 1:
            return ops.argmax_rows(logits)
        vals = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
        ids = ops.argmax_rows(logits, id_offset=self.w.vocab_shard[0], out_vals=vals)
        return self.comm.argmax_merge(vals, ids)

    def forward(self, b: ForwardBatch, kv: PagedKVCache, return_logits: bool = False,
                inputs_embeds: torch.Tensor | None = None) -> torch.Tensor:
        n = self.hidden_states(b, kv, inputs_embeds)
        lg = self.logits(n, b)
        if self.trace is not None:
            self.trace.record("logits", lg)
        if return_logits:
            return self.comm.all_gather_cat(lg) if self.w.tp.size > 1 else lg
        return self.greedy(lg)
