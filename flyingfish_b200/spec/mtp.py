"""Multi-token-prediction (MTP) speculation: the checkpoint's own extra layer drafts tokens, the
target verifies them in one batched forward.

An MTP module consumes, for position p, the target's final hidden state h_p and the embedding of
token p+1, ``x = eh_proj([enorm(emb(tok_{p+1})) | hnorm(h_p)])``, runs one decoder layer with its
own KV cache and predicts token p+2 through the shared head; deeper drafts feed the module's own
hidden state back in (depth 1-4, like the reference's chain, src/mtp.rs:12-66, 101-214).

A round is a transaction (src/mtp/batched.rs:71-194): draft k tokens (the first MTP row is
canonical, the rest speculative), verify k+1 rows with the target, accept the matching prefix plus
the bonus token, commit only accepted rows, then *repair* the MTP cache: rebuild the rows of the
accepted positions from the target's true hidden states. Output equals plain greedy decoding.
"""
from __future__ import annotations

import copy
import time
from dataclasses import dataclass

import torch

from .. import ops
from ..api import GenerationOutput, Model
from ..config import ModelSpec
from ..engine.batch import BatchLayout, ForwardBatch
from ..engine.kv_cache import PagedKVCache
from ..models.decoder import DecoderModel
from ..models.weights import DTYPES, ModelWeights, build_decoder_weights, synthetic_source
from .accept import accept_chain
from .chain import Fault, SpecFault, SpecStats

MAX_VERIFY_ROWS = 5          # depth <= 4 drafts + the pending token (src/mtp/batched.rs)


@dataclass
class MtpWeights:
    enorm: torch.Tensor
    hnorm: torch.Tensor
    eh_proj: torch.Tensor            # [hidden, 2*hidden]
    layer: ModelWeights              # one-layer decoder sharing embed / lm_head with the target


def build_mtp_weights(target_w: ModelWeights, source, device) -> MtpWeights:
    """Assemble the MTP module from a tensor source using the DeepSeek-V3 naming: the module lives
    at layer index ``num_hidden_layers`` with ``enorm / hnorm / eh_proj / shared_head.norm``."""
    spec = target_w.spec
    L = spec.layers
    one = copy.copy(spec)
    one.layers = 1
    one.mtp_layers = 0
    if one.moe is not None:
        one.moe = copy.copy(one.moe)
        one.moe.first_dense_layers = 0

    def remap(name: str, shape):
        if name.startswith("model.layers.0."):
            name = f"model.layers.{L}." + name[len("model.layers.0."):]
        elif name == "model.norm.weight":
            name = f"model.layers.{L}.shared_head.norm.weight"
        elif name in ("model.embed_tokens.weight", "lm_head.weight"):
            return None
        return source(name, shape)

    def src(name, shape):
        t = remap(name, shape)
        if t is None:       # shared with the target
            return target_w.embed if name == "model.embed_tokens.weight" else target_w.lm_head
        return t

    if spec.mla is not None:
        # DeepSeek-style targets: the module is a full MLA + MoE layer in the target's weight formats
        from ..models.deepseek import build_deepseek_weights
        layer = build_deepseek_weights(one, src, device, target_w.tp)
    else:
        layer = build_decoder_weights(one, src, device, target_w.tp)
    layer.embed, layer.lm_head, layer.vocab_shard = target_w.embed, target_w.lm_head, target_w.vocab_shard
    h = spec.hidden
    p = f"model.layers.{L}."
    return MtpWeights(enorm=source(p + "enorm.weight", (h,)), hnorm=source(p + "hnorm.weight", (h,)),
                      eh_proj=source(p + "eh_proj.weight", (h, 2 * h)), layer=layer)


class MtpSpeculator:
    """Single-sequence MTP speculation on top of a loaded target model."""

    def __init__(self, target: Model, depth: int = 2, seed: int = 0, weights: MtpWeights | None = None):
        if not 1 <= depth <= MAX_VERIFY_ROWS - 1:
            raise ValueError("MTP depth must be between 1 and 4")
        self.target, self.depth = target, depth
        te = target.engine
        tw = te.model.w
        dev = te.device
        if weights is None:
            weights = build_mtp_weights(tw, synthetic_source(tw.spec, seed, dev, DTYPES[tw.spec.dtype]), dev)
        self.w = weights
        spec = weights.layer.spec
        if spec.mla is not None:
            from ..models.deepseek import DeepseekModel
            self.net = DeepseekModel(weights.layer, comm=te.model.comm)
            self.kv = PagedKVCache(1, 1, spec.mla.kv_lora_rank + spec.mla.qk_rope_dim, te.max_blocks + 1,
                                   te.settings.kv_block, tw.embed.dtype, dev, v_head_dim=0)
        else:
            self.net = DecoderModel(weights.layer, comm=te.model.comm)
            hkv = max(1, spec.kv_heads // tw.tp.size)
            self.kv = PagedKVCache(1, hkv, spec.head_dim, te.max_blocks + 1, te.settings.kv_block, tw.embed.dtype, dev)
        self.fb = ForwardBatch(BatchLayout(1, max(te.max_prefill_rows, 8), te.max_blocks), dev)
        self.stats = SpecStats()
        self.fault = Fault.NONE

    # -- MTP forward over rows of one sequence ----------------------------------------------------
    def _mtp_rows(self, tokens: list[int], hidden: torch.Tensor, commit: int) -> tuple[list[int], torch.Tensor]:
        """Run the module on pairs (hidden[i], tokens[i]) at consecutive positions starting at the
        module cache's committed length; commit the first ``commit`` rows. Returns the greedy
        draft token and the module's final hidden state for every row."""
        rows = len(tokens)
        kvs = self.kv.seqs[0]
        slots = self.kv.reserve(0, rows)
        fb = self.fb
        fb.fill(ids=tokens, positions=list(range(kvs.length, kvs.length + rows)), slots=slots, q_lens=[rows],
                ctx_lens=[kvs.length + rows], block_rows=[list(kvs.blocks)], logit_rows=list(range(rows)),
                is_decode=False)
        fb.upload()
        w, spec = self.w, self.net.spec
        # [norm(embedding) | norm(previous hidden)] in one launch, then the mixing projection
        from ..ops import spec_ops
        x0 = ops.linear(spec_ops.mtp_mix(fb.ids, self.w.layer.embed, hidden.contiguous(), w.enorm, w.hnorm, spec.rms_eps),
                        w.eh_proj)
        n = self.net.hidden_states(fb, self.kv, inputs_embeds=x0)
        toks = self.net.greedy(self.net.logits(n, fb))
        self.kv.commit(0, commit)
        return [int(t) for t in toks.cpu().tolist()], n

    # -- generation ---------------------------------------------------------------------------------
    def generate(self, ids: list[int], count: int, ignore_eos: bool = True, on_tokens=None,
                 should_stop=None) -> GenerationOutput:
        """``on_tokens(list)`` receives every batch of emitted tokens (first token, then one call per round);
        ``should_stop()`` is polled between rounds (client disconnect)."""
        te = self.target.engine
        spec = self.target.spec
        eos = tuple(spec.extra.get("eos_token_ids", [spec.eos_token_id] if spec.eos_token_id is not None else []))
        if len(ids) + count + self.depth + 1 > te.settings.capacity:
            raise ValueError("prompt + output + verification rows exceed the KV capacity")
        if 0 in self.kv.seqs:
            self.kv.free_sequence(0)
        self.kv.add_sequence(0)
        t0 = time.perf_counter()
        ts = te.add_sequence(ids)
        sink: list = []
        te.model.normed_sink = sink
        try:
            first = te.prefill([ts])[0]
            te.model.normed_sink = None
            hid = torch.cat(sink, dim=0)                       # target hidden of every prompt position
            # MTP bootstrap: rows (h_p, tok_{p+1}) for the whole prompt except the last position
            if len(ids) > 1:
                self._mtp_rows(ids[1:], hid[:-1], commit=len(ids) - 1)
            h_prev = hid[-1:]
            out = [first]
            if on_tokens:
                on_tokens([first])
            t1 = time.perf_counter()
            while len(out) < count and not (not ignore_eos and eos and out[-1] in eos):
                if should_stop is not None and should_stop():
                    break
                k = min(self.depth, count - len(out))
                emitted, h_prev = self._round(ts, h_prev, k, eos, ignore_eos)
                emitted = emitted[: count - len(out)]
                out.extend(emitted)
                if on_tokens and emitted:
                    on_tokens(emitted)
            out = out[:count]
            t2 = time.perf_counter()
            return GenerationOutput(ids=out, prefill_ms=(t1 - t0) * 1e3, decode_ms=(t2 - t1) * 1e3,
                                    decode_steps=self.stats.rounds,
                                    extra={"verify": "batched", "accepted_per_round": self.stats.accepted_per_round,
                                           "acceptance_rate": self.stats.acceptance_rate})
        finally:
            te.model.normed_sink = None
            te.free_sequence(ts.seq_id)

    def _round(self, ts, h_prev: torch.Tensor, k: int, eos, ignore_eos: bool):
        te = self.target.engine
        base = self.kv.seqs[0].length
        if self.fault is Fault.DRAFT:
            raise SpecFault("injected draft failure")
        # ---- draft: row 0 pairs the TRUE hidden with the pending token (canonical), deeper rows
        # feed the module's own hidden back in (speculative); all are dropped or rebuilt below ----
        drafts: list[int] = []
        tok, h = ts.pending, h_prev
        for _ in range(k):
            d, hn = self._mtp_rows([tok], h, commit=1)
            drafts.append(d[0])
            tok, h = d[0], hn
        if self.fault is Fault.VERIFY:
            self.kv.truncate(0, base)
            raise SpecFault("injected verify failure")
        # ---- verify: one target forward of k+1 rows; keep its hidden states ----
        sink: list = []
        te.model.normed_sink = sink
        try:
            target_dev = te.verify([ts], [drafts], device_out=True)         # int32 [k + 1], still on the device
        except Exception:
            self.kv.truncate(0, base)
            raise
        finally:
            te.model.normed_sink = None
        true_h = sink[0]                                     # [k+1, hidden]
        # acceptance on the device; one small read-back carries the verdict
        from ..ops import spec_ops
        from .accept import Accepted
        d_dev = torch.tensor([drafts], dtype=torch.int32, device=target_dev.device)
        verdict = spec_ops.accept_chain(d_dev, target_dev.view(1, -1).to(torch.int32), eos, ignore_eos)[0].cpu().tolist()
        te._after_sync()
        acc = Accepted(verdict[3: 3 + verdict[1]], verdict[0], bool(verdict[2]))
        if self.fault is Fault.COMMIT:
            self.kv.truncate(0, base)
            raise SpecFault("injected commit failure")
        te.commit_verified(ts, acc.tokens, acc.n_draft_accepted)
        # ---- repair: keep the canonical row, rebuild the rows of the accepted drafts from the
        # target's true hidden states ----
        self.kv.truncate(0, base + 1)
        n = acc.n_draft_accepted
        if n > 0:
            self._mtp_rows(drafts[:n], true_h[:n], commit=n)
        st = self.stats
        st.rounds += 1; st.drafted += k; st.accepted += n; st.emitted += len(acc.tokens)
        st.accepted_per_round.append(n)
        return acc.tokens, true_h[n: n + 1]


def generate_mtp(model: Model, ids: list[int], count: int, depth: int = 2, ignore_eos: bool = True
                 ) -> GenerationOutput:
    spec = MtpSpeculator(model, depth=depth)
    return spec.generate(ids, count, ignore_eos)
