"""DeepSeek-V4.1-style decoder: manifold-constrained hyper-connections around every sublayer, a latent mixer with
one shared key/value head whose rows live in a per-sequence FP8 ring (window attention with a sink), top-k sparse
attention with a pooled indexer in the layers that compress, n-gram memory rows (Engram) added to the stream, and a
shared + routed expert FFN with square-root-soft-plus routing.

Layer program (the reference's nine-stage hyper-connection program, src/model.rs:440-520, and its latent mixer,
src/backend/cuda/engine_deepseek.rs:1119-1700; sparse layers: engine_deepseek_dsa.rs:545-1040, kernels/dsa.cu):

    stream [rows, mult, hidden]                                 ``mult`` residual copies per token
    (pre_a, post_a, comb_a) = mixes(stream)                     Sinkhorn-normalised combination matrix
    x   = collapse(stream, carried pre)                         carried = the previous layer's FFN pre (one-hot first)
    a   = mixer(rmsnorm(x))
    stream = update(a, stream, post_a, comb_a)
    (pre_f, post_f, comb_f) = mixes(stream)
    x   = collapse(stream, pre_a)                               the FFN stage collapses with the attention's own pre
    f   = ffn(rmsnorm(x))
    stream = update(f, stream, post_f, comb_f);  carried = pre_f
    ... after the last layer: rmsnorm(collapse(stream, carried)) -> lm_head

Mixer: q = wq_b(rmsnorm(wq_a n)) [heads, D]; k = rmsnorm(wkv n) [D] (one latent head, the value is the key content);
adjacent-pair rotary on the last ``rope_tail`` dims of q and k.
  * window layers: the key row is quantised (E4M3 codes, one E8M0 scale per 32) into slot ``position % ring`` of the
    sequence's ring; every query reads the ``window`` positions up to its own. The ring is ``window + chunk - 1`` slots
    long so that the rows of one prefill chunk (or of a speculative verification) never overwrite a slot a query of the
    same launch still reads.
  * sparse layers: the key row, an index key and a pooling logit row are appended to per-sequence BF16 tables; groups
    of four tokens are pooled into one index key; every query scores the pools of its sequence with 32 ReLU index heads,
    keeps the ``index_topk`` best and attends to their tokens plus the tokens after the last complete pool.
  both end with the inverse rotary on the output tail (window kernel: built in; sparse: the same pair kernel),
  a block-diagonal group projection ``wo_a`` and ``wo_b``.

Per-sequence state (rings, sparse tables, n-gram history) is addressed by the engine's state slots; the step is not
captured in a CUDA graph (host-side Engram row service runs inside it) and is not tensor-parallel.
"""
from __future__ import annotations

import math
import os
import tempfile
from dataclasses import dataclass

import numpy as np
import torch

from .. import ops
from ..config import ModelSpec
from ..ops import dsa_ops, latent_ops, mhc_ops, mla_ops
from .decoder import DecoderModel
from .deepseek import source_with_stub_attention
from .weights import ModelWeights, TPInfo, build_decoder_weights, random_tensor

BF16 = torch.bfloat16


@dataclass
class HcWeights:
    fn: torch.Tensor        # [(2 + mult) * mult, mult * hidden] bf16
    base: torch.Tensor      # [(2 + mult) * mult] f32
    scale: torch.Tensor     # [3] f32


@dataclass
class V41Weights:
    wq_a: torch.Tensor      # [q_lora, hidden]
    q_ln: torch.Tensor
    wq_b: torch.Tensor      # [heads * D, q_lora]
    wkv: torch.Tensor       # [D, hidden]
    kv_ln: torch.Tensor
    sink: torch.Tensor      # [heads] f32
    wo_a: torch.Tensor      # [groups, o_rank, heads / groups * D]
    wo_b: torch.Tensor      # [hidden, groups * o_rank]
    hc_attn: HcWeights
    hc_ffn: HcWeights
    # sparse layers only
    w_idx_q: torch.Tensor | None = None     # [32 * 128, q_lora]
    w_idx_w: torch.Tensor | None = None     # [32, hidden]
    w_idx_k: torch.Tensor | None = None     # [128, hidden]
    w_pool: torch.Tensor | None = None      # [128, hidden]
    ape: torch.Tensor | None = None         # [4, 128]
    # engram layers only
    w_engram: torch.Tensor | None = None    # [hidden, hash_width * 256]


def build_v41_weights(spec: ModelSpec, seed: int, device, source, tp: TPInfo | None = None, ep: TPInfo | None = None
                      ) -> ModelWeights:
    """FFN / norms / embeddings from the common builder; the mixer, hyper-connection, indexer and Engram projections are
    attached per layer as ``lw.extra['v41']``."""
    import copy
    c = spec.extra["v41"]
    stub = copy.copy(spec)
    stub.heads, stub.kv_heads, stub.head_dim, stub.qk_norm = 1, 1, 16, False
    w = build_decoder_weights(stub, source_with_stub_attention(source, device), device, tp, ep)
    w.spec = spec
    h, heads, d, mult = spec.hidden, spec.heads, spec.head_dim, int(c["hc_mult"])
    groups, o_rank, q_lora = int(c["o_groups"]), int(c["o_rank"]), int(c["q_lora"])
    dt = w.embed.dtype

    def rnd(name, shape, std=0.02, dtype=None):
        t = random_tensor(seed, name, shape, torch.float32, torch.device("cpu")) * (std / 0.02)
        return t.to(dtype or dt).contiguous().to(device)

    def hc(prefix):
        n = (2 + mult) * mult
        return HcWeights(rnd(prefix + "fn", (n, mult * h), 0.02, BF16), rnd(prefix + "base", (n,), 0.5, torch.float32),
                         torch.tensor([1.0, 1.0, 1.0], dtype=torch.float32, device=device))
    engram_layers = set((c.get("engram") or {}).get("layers", []))
    hash_width = 0
    if engram_layers:
        e = c["engram"]
        hash_width = (int(e["ngram"]) - 1) * int(e["heads"])
    for i, lw in enumerate(w.layers):
        p = f"model.layers.{i}.attn."
        lw.wqkv = None
        ones = torch.ones
        v = V41Weights(
            wq_a=rnd(p + "wq_a", (q_lora, h)), q_ln=ones(q_lora, dtype=dt, device=device),
            wq_b=rnd(p + "wq_b", (heads * d, q_lora), 0.05), wkv=rnd(p + "wkv", (d, h), 0.05),
            kv_ln=ones(d, dtype=dt, device=device), sink=rnd(p + "sink", (heads,), 0.5, torch.float32),
            wo_a=rnd(p + "wo_a", (groups, o_rank, heads // groups * d), 0.02, BF16), wo_b=rnd(p + "wo_b", (h, groups * o_rank)),
            hc_attn=hc(p + "hc."), hc_ffn=hc(f"model.layers.{i}.ffn.hc."))
        if i in set(c.get("sparse_layers", [])):
            v.w_idx_q = rnd(p + "indexer.wq", (dsa_ops.HEADS * dsa_ops.DIM, q_lora), 0.05)
            v.w_idx_w = rnd(p + "indexer.weights", (dsa_ops.HEADS, h), 0.05)
            v.w_idx_k = rnd(p + "indexer.wk", (dsa_ops.DIM, h), 0.05)
            v.w_pool = rnd(p + "compressor.wgate", (dsa_ops.DIM, h), 0.05)
            v.ape = rnd(p + "compressor.ape", (dsa_ops.POOL, dsa_ops.DIM), 0.1, BF16)
        if i in engram_layers:
            v.w_engram = rnd(f"model.layers.{i}.engram.proj", (h, hash_width * 256), 0.01)
        lw.extra["v41"] = v
        lw.wo = v.wo_b
    return w


class DeepseekV41Model(DecoderModel):
    owns_token_state = True          # rings and sparse tables live here; the engine's block cache only counts positions

    def __init__(self, weights: ModelWeights, comm=None, trace=None, max_sequences: int = 64, max_len: int = 4096,
                 max_chunk: int = 256, seed: int = 0, runtime_dir: str | None = None):
        super().__init__(weights, comm=comm, trace=trace)
        assert weights.tp.size == 1, "the latent mixer is not tensor-parallel"
        c = self.spec.extra["v41"]
        self.c = c
        self.mult, self.window, self.rope_tail = int(c["hc_mult"]), int(c["window"]), int(c["rope_tail"])
        self.hc_iters, self.hc_eps = int(c.get("hc_iters", 3)), float(c.get("hc_eps", 1e-6))
        self.groups = int(c["o_groups"])
        self.index_topk = int(c.get("index_topk", dsa_ops.TOPK))
        self.sparse_layers = set(c.get("sparse_layers", []))
        # which pre-mix collapses the stream before a sublayer: "carried" (DeepSeek: the attention stage uses the
        # previous layer's FFN pre, the FFN stage the attention's own) or "own" (GLM: every stage its own, nothing
        # carried across layers) -- src/model.rs:459-482 of the reference
        self.hc_policy = str(c.get("hc_policy", "carried"))
        assert self.hc_policy in ("carried", "own")
        self.prefill_take_limit = max_chunk                      # rows of one sequence per launch (ring headroom)
        self.ring = self.window + max_chunk - 1
        self.max_len = (max_len + dsa_ops.POOL - 1) // dsa_ops.POOL * dsa_ops.POOL
        self.state_slot_count = max_sequences + 1
        dev, d, n = weights.embed.device, self.d, self.state_slot_count
        self.codes = {i: torch.zeros(n, self.ring, d, dtype=torch.uint8, device=dev)
                      for i in range(self.spec.layers) if i not in self.sparse_layers}
        self.scales = {i: torch.zeros(n, self.ring, d // 32, dtype=torch.uint8, device=dev) for i in self.codes}
        rows = n * self.max_len
        self.latent = {i: torch.zeros(rows, d, dtype=BF16, device=dev) for i in self.sparse_layers}
        self.idx_key = {i: torch.zeros(rows, dsa_ops.DIM, dtype=BF16, device=dev) for i in self.sparse_layers}
        self.pool_logit = {i: torch.zeros(rows, dsa_ops.DIM, dtype=BF16, device=dev) for i in self.sparse_layers}
        self.pooled = {i: torch.zeros(rows // dsa_ops.POOL, dsa_ops.DIM, dtype=BF16, device=dev) for i in self.sparse_layers}
        self._meta = None
        self._init_engram(seed, runtime_dir)

    # -- Engram ------------------------------------------------------------------------------------
    def _init_engram(self, seed: int, runtime_dir: str | None) -> None:
        e = self.c.get("engram")
        self.engram = None
        if not e:
            return
        from ..engram import ROW_BYTES, EngramHashSetup, NgramHistory, RowService
        layers = list(e["layers"])
        setup = EngramHashSetup.build(layers, self.spec.vocab, int(e["compressed_vocab"]), int(e["ngram"]), int(e["heads"]),
                                      int(e["table_rows"]), seed=seed)
        # random-init shapes carry a generated table file (codes + power-of-two scales) per Engram layer
        root = runtime_dir or tempfile.mkdtemp(prefix="ff_engram_")
        services = []
        for li, layer in enumerate(layers):
            rows = setup.table_rows(li)
            path = os.path.join(root, f"engram_{self.spec.name}_{layer}_{seed}.bin")
            if not os.path.exists(path) or os.path.getsize(path) != rows * ROW_BYTES:
                rng = np.random.default_rng(seed * 1000 + layer)
                tab = np.empty((rows, ROW_BYTES), dtype=np.uint8)
                tab[:, :256] = rng.integers(-64, 64, size=(rows, 256), dtype=np.int8).view(np.uint8)
                tab[:, 256:] = rng.integers(118, 122, size=(rows, 8), dtype=np.uint8)
                tab.tofile(path)
            services.append(RowService(path, rows, int(e.get("cache_rows", 4096))))
        self.engram = {"setup": setup, "layers": layers, "services": services,
                       "history": [NgramHistory(setup, self.max_len) for _ in range(self.state_slot_count)]}

    def _engram_rows(self, b) -> dict[int, torch.Tensor]:
        """Per Engram layer, the decoded memory rows of this batch [rows, hash_width * 256] (host service)."""
        from ..engram import decode_rows
        L = b.layout
        rows = b.rows
        ids = b.host[L.ids: L.ids + rows].tolist()
        pos = b.host[L.positions: L.positions + rows].tolist()
        lens = b.host[L.q_lens: L.q_lens + b.batch].tolist() if not b.is_decode else [b.nq] * b.batch
        eg = self.engram
        per_layer: list[list[int]] = [[] for _ in eg["layers"]]
        r = 0
        for s, n in enumerate(lens):
            slot = self._slots_host[s]
            if slot == self.state_slot_count - 1:            # padding rows of a decode bucket: row 0 of every table
                width = eg["setup"].hash_width()
                for li in range(len(per_layer)):
                    per_layer[li] += [0] * (n * width)
            else:
                got = eg["history"][slot].prepare(ids[r: r + n], pos[r])
                for li in range(len(per_layer)):
                    per_layer[li] += got[li]
            r += n
        out = {}
        dev, dt = self.w.embed.device, self.w.embed.dtype
        for li, layer in enumerate(eg["layers"]):
            raw = eg["services"][li].gather(per_layer[li])
            vals = decode_rows(raw).reshape(rows, -1)
            out[layer] = torch.from_numpy(vals).to(dt).to(dev, non_blocking=True)
        return out

    # -- per-sequence state ---------------------------------------------------------------------------
    def reset_state(self, slot: int) -> None:
        for i in self.codes:
            self.codes[i][slot].zero_()
            self.scales[i][slot].zero_()
        if self.engram is not None:
            self.engram["history"][slot].reset()
        # the sparse tables are addressed by position and overwritten before they are read: nothing to clear

    def state_bytes_per_sequence(self) -> int:
        d = self.d
        return (len(self.codes) * self.ring * (d + d // 32)
                + len(self.sparse_layers) * self.max_len * 2 * (d + 2 * dsa_ops.DIM + dsa_ops.DIM // dsa_ops.POOL))

    def state_tables(self) -> list[torch.Tensor]:
        """Every per-token table of the sparse layers (for :func:`dsa_ops.checkpoint_save`)."""
        t = []
        for i in sorted(self.sparse_layers):
            t += [self.latent[i], self.idx_key[i], self.pool_logit[i]]
        return t

    # -- forward ------------------------------------------------------------------------------------
    def _prepare(self, b) -> None:
        dev = self.w.embed.device
        slots = list(getattr(b, "state_slots", None) or [])
        assert len(slots) == b.batch, "the engine must name a state slot per sequence of the batch"
        self._slots_host = slots
        L = b.layout
        lens = [b.nq] * b.batch if b.is_decode else b.host[L.q_lens: L.q_lens + b.batch].tolist()
        assert max(lens) <= self.prefill_take_limit, "more rows of one sequence than the ring headroom allows"
        slot_t = torch.tensor(slots, dtype=torch.int32, device=dev)
        len_t = torch.tensor(lens, dtype=torch.int64, device=dev)
        row_slot = torch.repeat_interleave(slot_t, len_t)
        pad = b.rows - row_slot.numel()
        if pad > 0:                                               # rows that belong to no sequence
            row_slot = torch.cat([row_slot, torch.full((pad,), self.state_slot_count - 1, dtype=torch.int32, device=dev)])
        pos = b.positions
        m = {"row_slot": row_slot.contiguous(), "seq_base": (row_slot * self.max_len).to(torch.int32).contiguous(),
             "cs": latent_ops.rotary_table(pos, self.rope_tail, self.spec.rope_theta),
             "inv": latent_ops.rotary_table(pos, self.rope_tail, self.spec.rope_theta, inverse=True)}
        if self.sparse_layers:
            # pools completed by this launch, per sequence: [first_new, first_new + n_new)
            first_pos = b.host[L.positions: L.positions + b.rows].tolist()
            st, ln, dst, r = [], [], [], 0
            for s, n in enumerate(lens):
                p0, p1 = first_pos[r], first_pos[r] + n
                a, z = p0 // dsa_ops.POOL, p1 // dsa_ops.POOL
                if z > a and slots[s] != self.state_slot_count - 1:
                    base = slots[s] * self.max_len
                    st.append(base + a * dsa_ops.POOL)
                    ln.append((z - a) * dsa_ops.POOL)
                    dst += list(range(base // dsa_ops.POOL + a, base // dsa_ops.POOL + z))
                r += n
            m["pool_new"] = None
            if st:
                m["pool_new"] = (torch.tensor(st, dtype=torch.int32, device=dev), torch.tensor(ln, dtype=torch.int32, device=dev),
                                 torch.tensor(dst, dtype=torch.long, device=dev))
            m["global_row"] = (m["seq_base"].long() + pos.long())
            m["pool_base"] = (m["seq_base"] // dsa_ops.POOL).to(torch.int32).contiguous()
            m["n_cand"] = ((pos + 1) // dsa_ops.POOL).to(torch.int32).contiguous()
        self._meta = m

    def _hc(self, stream: torch.Tensor, hw: HcWeights):
        return mhc_ops.mixes(stream, hw.fn, hw.base, hw.scale, self.hc_iters, self.hc_eps, self.spec.rms_eps)

    def _mixer(self, i: int, n: torch.Tensor, b) -> torch.Tensor:
        s, m = self.spec, self._meta
        v: V41Weights = self.w.layers[i].extra["v41"]
        rows, heads, d = n.shape[0], s.heads, self.d
        qa = ops.rmsnorm(ops.linear(n, v.wq_a), v.q_ln, s.rms_eps)
        q = ops.linear(qa, v.wq_b)
        k = ops.rmsnorm(ops.linear(n, v.wkv), v.kv_ln, s.rms_eps)
        if q.dtype != BF16:
            q, k = q.to(BF16), k.to(BF16)
        latent_ops.rope_pair_tail(q, m["cs"], heads, d, self.rope_tail)
        latent_ops.rope_pair_tail(k, m["cs"], 1, d, self.rope_tail)
        q3 = q.view(rows, heads, d)
        if i not in self.sparse_layers:
            latent_ops.ring_write(k, m["row_slot"], b.positions, self.codes[i], self.scales[i])
            a = latent_ops.window_attention(q3, self.codes[i], self.scales[i], m["row_slot"], b.positions, v.sink,
                                            self.rope_tail, s.rope_theta, scale=self.scale, visible=self.window,
                                            inv_rot=m["inv"])
        else:
            g = m["global_row"]
            self.latent[i].index_copy_(0, g, k)
            self.idx_key[i].index_copy_(0, g, ops.linear(n, v.w_idx_k).to(BF16))
            self.pool_logit[i].index_copy_(0, g, ops.linear(n, v.w_pool).to(BF16))
            if m["pool_new"] is not None:
                st, ln, dst = m["pool_new"]
                pooled, _ = dsa_ops.pool_keys(self.idx_key[i], self.pool_logit[i], v.ape, st, ln)
                self.pooled[i].index_copy_(0, dst, pooled)
            iq = ops.linear(qa, v.w_idx_q).to(BF16).view(rows, dsa_ops.HEADS, dsa_ops.DIM).contiguous()
            iw = ops.linear(n, v.w_idx_w).to(BF16).contiguous()
            sel, _ = dsa_ops.index_topk(iq, iw, self.pooled[i], m["pool_base"], m["n_cand"], k=self.index_topk)
            idx = dsa_ops.expand(sel, m["seq_base"], b.positions)
            a = dsa_ops.sparse_attention(q3.contiguous(), self.latent[i], idx, v.sink, scale=self.scale)
            a2 = a.view(rows, heads * d)
            latent_ops.rope_pair_tail(a2, m["inv"], heads, d, self.rope_tail)
        if self.trace is not None:
            self.trace.record(f"layer.{i}.attn", a)
        og = mla_ops.per_head_linear(a.view(rows, self.groups, heads // self.groups * d), v.wo_a)   # [rows, groups, o_rank]
        return ops.linear(og.reshape(rows, -1).to(v.wo_b.dtype), v.wo_b)

    def hidden_states(self, b, kv, inputs_embeds=None):
        w, s = self.w, self.spec
        self._prepare(b)
        x = ops.embed(b.ids, w.embed) if inputs_embeds is None else inputs_embeds
        rows, mult = x.shape[0], self.mult
        memory = self._engram_rows(b) if self.engram is not None else {}
        stream = x.to(BF16)[:, None, :].expand(rows, mult, s.hidden).contiguous()
        carried = torch.zeros(rows, mult, dtype=torch.float32, device=x.device)
        carried[:, 0] = 1.0
        dt = w.embed.dtype
        for i in range(s.layers):
            lw = w.layers[i]
            v: V41Weights = lw.extra["v41"]
            if i in memory:
                # n-gram memory rows enter every residual copy through one projection
                mem = ops.linear(memory[i], v.w_engram).to(BF16)
                stream = (stream.float() + mem.float()[:, None, :]).to(BF16)
            pre_a, post_a, comb_a = self._hc(stream, v.hc_attn)
            xa = mhc_ops.collapse(stream, carried if self.hc_policy == "carried" else pre_a).to(dt)
            a = self._mixer(i, ops.rmsnorm(xa, lw.input_ln, s.rms_eps), b)
            stream = mhc_ops.update(a.to(BF16), stream, post_a, comb_a)
            pre_f, post_f, comb_f = self._hc(stream, v.hc_ffn)
            xf = mhc_ops.collapse(stream, pre_a if self.hc_policy == "carried" else pre_f).to(dt)
            f = self._ffn(i, ops.rmsnorm(xf, lw.post_ln, s.rms_eps))
            stream = mhc_ops.update(f.to(BF16), stream, post_f, comb_f)
            carried = pre_f
            if self.trace is not None:
                self.trace.record(f"layer.{i}", stream)
        out = mhc_ops.collapse(stream, carried).to(dt)
        n = ops.rmsnorm(out, w.final_norm, s.rms_eps)
        self.last_residual = out
        if self.normed_sink is not None:
            self.normed_sink.append(n)
        return n
