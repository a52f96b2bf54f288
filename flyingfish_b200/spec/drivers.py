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


# ------------------------------------------------------------------------------------------------
# Draft-model ("DSpark") tools: replay-draft, replay-tree, check-tree-greedy, compare-tree-builders,
# compare-tree-padding, compare-spec-graph (src/spec.rs:472-990, src/tree_replay.rs:90). Every tool
# runs on a seeded prompt, returns one JSON object, and never changes what greedy decoding would emit.
# ------------------------------------------------------------------------------------------------
def _prompt(model, n: int) -> list[int]:
    g = torch.Generator().manual_seed(1)
    return torch.randint(0, model.spec.vocab, (n,), generator=g).tolist()


def _plain(model, ids, n):
    out = generate_plain(model, ids, n, ignore_eos=True, graph=False)
    model.reset()
    return out


def _record_chain(target, draft, ids, n, k: int = 4) -> dict:
    """Run chain speculation and record every round: the draft tokens, the target's tokens, what was accepted."""
    from .chain import ChainSpeculator
    sp = ChainSpeculator(target, draft, k=k)
    rounds: list[dict] = []
    orig = sp._round

    def spy(ts, ds, kk, eos, ignore_eos):
        before = len(sp.stats.accepted_per_round)
        emitted = orig(ts, ds, kk, eos, ignore_eos)
        rounds.append({"k": kk, "accepted": sp.stats.accepted_per_round[before], "emitted": list(emitted)})
        return emitted
    sp._round = spy
    out = sp.generate(ids, n)
    target.reset(); draft.reset()
    return {"ids": out.ids, "rounds": rounds, "stats": sp.stats, "decode_ms": out.decode_ms}


def _record_tree(target, draft, ids, n, budget: str, builder: str) -> dict:
    from .tree_spec import TreeSpeculator
    sp = TreeSpeculator(target, draft, budget=budget, builder=builder)
    t0 = time.perf_counter()
    out = sp.generate(ids, n)
    dt = (time.perf_counter() - t0) * 1e3
    target.reset(); draft.reset()
    return {"ids": out.ids, "accepted_per_round": list(sp.stats.accepted_per_round), "stats": sp.stats, "ms": dt,
            "rows": sp.rows, "draft_forwards": sp.draft_forwards}


def run_dspark_tool(tool: str, target, draft, prompt_tokens: int, max_new_tokens: int, budget: str = "tree16",
                    builder: str = "waves", trace_path: str | None = None, strict: bool = False) -> dict:
    import json
    from pathlib import Path
    ids = _prompt(target, prompt_tokens)
    plain = _plain(target, ids, max_new_tokens)
    res: dict = {"tool": tool, "prompt_tokens": prompt_tokens, "max_new_tokens": max_new_tokens}

    if tool == "replay-draft":
        # record a chain-speculation run; when a trace file exists, replay must reproduce it round by round
        rec = _record_chain(target, draft, ids, max_new_tokens)
        trace = {"ids": rec["ids"], "rounds": rec["rounds"]}
        res.update(identical_to_greedy=rec["ids"] == plain.ids, rounds=len(rec["rounds"]),
                   acceptance_rate=rec["stats"].acceptance_rate)
        if trace_path and Path(trace_path).exists():
            old = json.loads(Path(trace_path).read_text())
            res["replay_matches_trace"] = old == trace
        elif trace_path:
            Path(trace_path).write_text(json.dumps(trace))
            res["trace_written"] = trace_path
    elif tool == "replay-tree":
        rec = _record_tree(target, draft, ids, max_new_tokens, budget, builder)
        trace = {"ids": rec["ids"], "accepted_per_round": rec["accepted_per_round"], "budget": budget, "builder": builder}
        res.update(identical_to_greedy=rec["ids"] == plain.ids, rounds=len(rec["accepted_per_round"]))
        if trace_path and Path(trace_path).exists():
            res["replay_matches_trace"] = json.loads(Path(trace_path).read_text()) == trace
        elif trace_path:
            Path(trace_path).write_text(json.dumps(trace))
            res["trace_written"] = trace_path
    elif tool == "check-tree-greedy":
        rec = _record_tree(target, draft, ids, max_new_tokens, budget, builder)
        res.update(identical_to_greedy=rec["ids"] == plain.ids, rounds=len(rec["accepted_per_round"]),
                   tokens_per_round=rec["stats"].tokens_per_round, budget=budget, builder=builder)
    elif tool == "compare-tree-builders":
        runs = {b: _record_tree(target, draft, ids, max_new_tokens, budget, b) for b in ("waves", "serial", "markov")}
        res.update(budget=budget, identical_to_greedy=all(r["ids"] == plain.ids for r in runs.values()),
                   builders={b: {"rounds": len(r["accepted_per_round"]), "tokens_per_round": r["stats"].tokens_per_round,
                                 "ms": r["ms"], "draft_forwards": r["draft_forwards"]} for b, r in runs.items()})
    elif tool == "compare-tree-padding":
        # the same run under every verification-row budget: more rows cost more per round and accept more per round
        runs = {b: _record_tree(target, draft, ids, max_new_tokens, b, builder) for b in ("tree16", "tree32", "tree64")}
        res.update(builder=builder, identical_to_greedy=all(r["ids"] == plain.ids for r in runs.values()),
                   budgets={b: {"rows": r["rows"], "rounds": len(r["accepted_per_round"]),
                                "tokens_per_round": r["stats"].tokens_per_round, "ms": r["ms"]} for b, r in runs.items()})
    elif tool == "compare-spec-graph":
        # draft model decoding from CUDA graphs against eager launches: same tokens, different time
        runs = {}
        for graph in (False, True):
            draft.engine.use_graph = graph and draft.engine.device.type == "cuda"
            r = _record_chain(target, draft, ids, max_new_tokens)
            runs["graph" if graph else "eager"] = {"ids": r["ids"], "decode_ms": r["decode_ms"], "rounds": len(r["rounds"])}
        res.update(identical=runs["graph"]["ids"] == runs["eager"]["ids"],
                   identical_to_greedy=runs["eager"]["ids"] == plain.ids,
                   eager_ms=runs["eager"]["decode_ms"], graph_ms=runs["graph"]["decode_ms"])
    else:
        raise ValueError(f"unknown tool {tool}")
    if strict and not res.get("identical_to_greedy", True):
        raise SystemExit(f"{tool}: speculative output differs from plain greedy decoding")
    return res
