"""Whole-sequence (non-autoregressive) use of the decoder stack: text encoders and masked-diffusion language
models. A model whose spec carries ``extra["bidirectional"]`` attends in both directions inside a sequence (the
paged prefill kernel in bidirectional mode), so every sequence must go through the stack in ONE chunk; nothing is
decoded and the KV blocks are released right after the pass.

Reference counterparts: the embedding path (``embed`` subcommand, kernels/embed.cu mean_pool_l2 / l2_normalize,
EmbeddingGemma2 in src/model_spec.rs:8-104) and the diffusion language models (Clover, DiffusionGemma canvas).
"""
from __future__ import annotations

import torch

from .. import ops


def run_whole(model, seqs_ids: list[list[int]], want: str = "hidden") -> list[torch.Tensor]:
    """One forward over whole sequences packed row-wise. ``want``: "hidden" -> final-normed rows [len, hidden] per
    sequence; "logits" -> [len, vocab] per sequence (FP32 on the host side of the call is the caller's choice)."""
    eng = model.engine
    total = sum(len(s) for s in seqs_ids)
    if total > eng.max_prefill_rows or len(seqs_ids) > eng.max_batch:
        raise ValueError(f"{total} rows / {len(seqs_ids)} sequences exceed one prefill chunk "
                         f"({eng.max_prefill_rows} rows, {eng.max_batch} sequences)")
    seqs = [eng.add_sequence(ids) for ids in seqs_ids]
    try:
        fb = eng.prefill_batch
        ids, positions, slots, q_lens, ctx_lens, block_rows = [], [], [], [], [], []
        for s in seqs:
            n = len(s.prompt)
            sl = eng.kv.reserve(s.seq_id, n)
            ids += s.prompt
            positions += list(range(n))
            slots += sl
            q_lens.append(n)
            ctx_lens.append(n)
            block_rows.append(list(eng.kv.seqs[s.seq_id].blocks))
        fb.fill(ids=ids, positions=positions, slots=slots, q_lens=q_lens, ctx_lens=ctx_lens, block_rows=block_rows,
                logit_rows=list(range(total)) if want == "logits" else [total - 1], is_decode=False,
                state_slots=[s.state_slot for s in seqs] if eng.state_slots is not None else None)
        fb.upload()
        fb.state_slots = [s.state_slot for s in seqs]      # models with per-sequence recurrent state address it by slot
        net = eng.model
        if want == "logits":
            out = net.forward(fb, eng.kv, return_logits=True)
        else:
            out = net.hidden_states(fb, eng.kv)
        parts, o = [], 0
        for n in q_lens:
            parts.append(out[o: o + n])
            o += n
        return parts
    finally:
        for s in seqs:
            eng.free_sequence(s.seq_id)


class EmbeddingHead:
    """Mean pooling over the sequence, optional dense layers (``extra["embed_dense"]`` = widths of successive
    bias-free linear layers, as in EmbeddingGemma's 768 -> 3072 -> 768 head), L2 normalisation."""

    def __init__(self, spec, device, seed: int = 0, state: dict[str, torch.Tensor] | None = None):
        widths = list(spec.extra.get("embed_dense") or [])
        g = torch.Generator().manual_seed(seed + 77)
        self.layers = []
        prev = spec.hidden
        for i, wd in enumerate(widths):
            w = state[f"dense.{i}.weight"] if state is not None else torch.randn(wd, prev, generator=g) * 0.02
            dt = torch.bfloat16 if torch.device(device).type == "cuda" else torch.float32
            self.layers.append(w.to(dt).contiguous().to(device))
            prev = wd
        self.out_dim = prev

    def __call__(self, hidden: torch.Tensor) -> torch.Tensor:
        v = hidden.float().mean(dim=0, keepdim=True)
        for w in self.layers:
            v = ops.linear(v.to(w.dtype).contiguous(), w).float()
        v = v[0]
        return v / v.norm().clamp_min(1e-12)


def embed_texts(model, texts_ids: list[list[int]], head: EmbeddingHead | None = None) -> list[torch.Tensor]:
    """Unit-length embedding of each token sequence (batched into as few whole-sequence passes as fit)."""
    eng = model.engine
    head = head or EmbeddingHead(model.spec, eng.device)
    out: list[torch.Tensor] = []
    batch: list[list[int]] = []
    rows = 0
    for ids in texts_ids + [None]:
        if ids is None or rows + len(ids) > eng.max_prefill_rows or len(batch) == eng.max_batch:
            if batch:
                out += [head(h) for h in run_whole(model, batch, "hidden")]
            batch, rows = [], 0
        if ids is not None:
            batch.append(ids)
            rows += len(ids)
    return out
