"""Masked-diffusion text generation: a canvas of mask tokens after the prompt is denoised in ``steps`` passes of a
bidirectional model; each pass predicts every position and commits the most confident predictions among the still
masked ones (confidence = probability of the arg-max token; ties go to the earlier position, arg-max ties to the
lower token id), so that all positions are committed after the last pass. With ``block`` the canvas is denoised
block by block from left to right (semi-autoregressive), each block with its own share of the steps.

Reference counterpart: the diffusion language models of the reference's model list (Clover, DiffusionGemma canvas;
src/model_spec.rs:8-104)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

from ..models.encoder import run_whole


@dataclass
class DiffusionTrace:
    committed_per_step: list[list[int]] = field(default_factory=list)     # canvas positions committed in each pass
    passes: int = 0


def diffusion_generate(model, prompt: list[int], length: int, steps: int, mask_id: int | None = None,
                       block: int | None = None, trace: DiffusionTrace | None = None) -> list[int]:
    if mask_id is None:
        mask_id = int(model.spec.extra["mask_token_id"])
    if length <= 0 or steps <= 0:
        raise ValueError("length and steps must be positive")
    block = block or length
    canvas = [mask_id] * length
    n_blocks = math.ceil(length / block)
    steps_per_block = max(1, steps // n_blocks)
    for bi in range(n_blocks):
        lo, hi = bi * block, min(length, (bi + 1) * block)
        for step in range(steps_per_block):
            masked = [i for i in range(lo, hi) if canvas[i] == mask_id]
            if not masked:
                break
            # later blocks stay masked and visible: the model sees the whole canvas every pass
            logits = run_whole(model, [prompt + canvas], "logits")[0][len(prompt):].float().cpu()
            logits[:, mask_id] = -math.inf                       # a position is never committed to the mask token
            probs = torch.softmax(logits, dim=-1)
            conf, tok = probs.max(dim=-1)                        # torch.max returns the first maximal index
            quota = math.ceil(len(masked) / (steps_per_block - step))
            order = sorted(masked, key=lambda i: (-float(conf[i]), i))[:quota]
            for i in order:
                canvas[i] = int(tok[i])
            if trace is not None:
                trace.committed_per_step.append(sorted(order))
                trace.passes += 1
    return canvas
