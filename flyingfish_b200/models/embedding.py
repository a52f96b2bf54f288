"""Text embeddings: mean-pooled, L2-normalised final hidden states (the reference's ``embed``
subcommand and its ``mean_pool_l2`` / ``l2_normalize`` kernels, kernels/embed.cu)."""
from __future__ import annotations

import torch


def embed_text(model, ids: list[int]) -> list[float]:
    eng = model.engine
    seq = eng.add_sequence(ids)
    sink: list = []
    eng.model.normed_sink = sink
    try:
        eng.prefill([seq])
    finally:
        eng.model.normed_sink = None
        eng.free_sequence(seq.seq_id)
    h = torch.cat(sink, dim=0).to(torch.float32)
    v = h.mean(dim=0)
    v = v / v.norm().clamp_min(1e-12)
    return [float(x) for x in v.cpu().tolist()]
