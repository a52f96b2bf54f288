"""Speculative-decoding tools behind ``ff verify-spec | bench-spec | profile-spec``: run MTP (or a
draft model) speculation, check the emitted stream against plain greedy decoding (``--strict``
fails on any difference) and report acceptance statistics as JSON (src/spec.rs:22-380, 644-800)."""
from __future__ import annotations

import time

import torch

from ..api import generate_plain


def run_spec_tool(tool: str, model, prompt_tokens: int, max_new_tokens: int, depth: int, strict: bool) -> dict:
    from .mtp import MtpSpeculator
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, model.spec.vocab, (prompt_tokens,), generator=g).tolist()
    plain = generate_plain(model, ids, max_new_tokens, ignore_eos=True, graph=False)
    model.reset()
    spec = MtpSpeculator(model, depth=depth)
    cuda = model.engine.device.type == "cuda"
    if tool == "profile-spec" and cuda:
        torch.cuda.profiler.start(); torch.cuda.nvtx.range_push("ff.spec")
    t0 = time.perf_counter()
    out = spec.generate(ids, max_new_tokens)
    dt = time.perf_counter() - t0
    if tool == "profile-spec" and cuda:
        torch.cuda.nvtx.range_pop(); torch.cuda.profiler.stop()
    same = out.ids == plain.ids
    if strict and not same:
        raise SystemExit("speculative output differs from plain greedy decoding")
    st = spec.stats
    return {"tool": tool, "identical_to_greedy": same, "rounds": st.rounds, "drafted": st.drafted,
            "accepted": st.accepted, "acceptance_rate": st.acceptance_rate, "tokens_per_round": st.tokens_per_round,
            "spec_ms": dt * 1e3, "plain_decode_ms": plain.decode_ms, "mtp_depth": depth}
