"""Tree speculation: a draft model proposes a token tree, the target verifies all of its rows in
one forward under ancestor masks, the best matching path is committed and its K/V rows are
compacted (the reference's tree round: src/backend/cuda/engine.rs:5893-6085, 4820-5190)."""
from __future__ import annotations

import time

import torch

from ..api import GenerationOutput, Model
from .accept import accept_tree
from .chain import SpecStats
from .tree import BUDGETS, build_tree


class TreeSpeculator:
    def __init__(self, target: Model, draft: Model, budget: str = "tree16", builder: str = "waves"):
        assert budget in BUDGETS and BUDGETS[budget] > 0
        self.target, self.draft = target, draft
        self.rows, self.builder = BUDGETS[budget], builder
        self.stats = SpecStats()

    def _children_fn(self, ds):
        de = self.draft.engine

        def fn(paths: list[list[int]]):
            outs = []
            for p in paths:
                logits = de.forward_rows(ds, p, return_logits=True)[-1].float()
                lp = torch.log_softmax(logits, dim=-1)
                v, i = torch.topk(lp, 4)
                outs.append([(int(t), float(x)) for t, x in zip(i.tolist(), v.tolist())])
            return outs
        return fn

    def generate(self, ids: list[int], count: int, ignore_eos: bool = True) -> GenerationOutput:
        te, de = self.target.engine, self.draft.engine
        if len(ids) + count + self.rows + 1 > te.settings.capacity:
            raise ValueError("prompt + output + tree rows exceed the KV capacity")
        t0 = time.perf_counter()
        ts, ds = te.add_sequence(ids), de.add_sequence(ids)
        try:
            first = te.prefill([ts])[0]
            de.prefill([ds])
            out = [first]
            t1 = time.perf_counter()
            while len(out) < count:
                tree = build_tree(ts.pending, self._children_fn(ds), self.rows, self.builder)
                target = te.verify_tree(ts, tree.tokens, tree.depth, tree.masks)
                acc, path = accept_tree(tree.parents, tree.tokens, target)
                te.commit_tree_path(ts, path, acc.tokens)
                # draft cache: commit the same tokens (pending + accepted) by a causal forward
                consumed = [tree.tokens[r] for r in path]
                de.forward_rows(ds, consumed, return_logits=False)
                de.kv.commit(ds.seq_id, len(consumed))
                out.extend(acc.tokens)
                st = self.stats
                st.rounds += 1; st.drafted += len(tree) - 1; st.accepted += acc.n_draft_accepted
                st.emitted += len(acc.tokens); st.accepted_per_round.append(acc.n_draft_accepted)
            t2 = time.perf_counter()
            return GenerationOutput(ids=out[:count], prefill_ms=(t1 - t0) * 1e3, decode_ms=(t2 - t1) * 1e3,
                                    decode_steps=self.stats.rounds,
                                    extra={"accepted_per_round": self.stats.accepted_per_round})
        finally:
            te.free_sequence(ts.seq_id)
            de.free_sequence(ds.seq_id)
