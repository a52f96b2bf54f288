"""Tree speculation: a draft model proposes a token tree, the target verifies all of its rows in
one forward under ancestor masks, the best matching path is committed and its K/V rows are
compacted (the reference's tree round: src/backend/cuda/engine.rs:5893-6085, 4820-5190).

Builders: ``waves`` / ``serial`` ask the draft model for the children of every expanded node (one draft forward per
node). ``markov`` is the block drafter's scheme (src/dspark.rs:892-950, kernels/markov.cu:1-55): the draft model runs
ONCE per depth along its own greedy chain, giving one base-logit row per depth; the children of any node at depth d are
the top-4 of ``bf16(w2 . w1[parent token]) + base[d]`` (a rank-256 bigram correction of the base distribution), all
nodes of a wave in one batched Markov-head launch."""
from __future__ import annotations

import time

import torch

from ..api import GenerationOutput, Model
from .accept import accept_tree
from .chain import SpecStats
from .tree import BUDGETS, build_tree


MARKOV_RANK, MARKOV_DEPTH = 256, 6


class TreeSpeculator:
    def __init__(self, target: Model, draft: Model, budget: str = "tree16", builder: str = "waves",
                 markov: tuple[torch.Tensor, torch.Tensor] | None = None, seed: int = 0):
        assert budget in BUDGETS and BUDGETS[budget] > 0
        assert builder in ("waves", "serial", "markov")
        self.target, self.draft = target, draft
        self.rows, self.builder = BUDGETS[budget], builder
        self.stats = SpecStats()
        self.draft_forwards = 0
        self.markov = markov
        if builder == "markov" and markov is None:
            # no trained head at hand: a seeded low-rank pair (a head shipped with a draft checkpoint replaces it)
            g = torch.Generator().manual_seed(seed + 977)
            dev = draft.engine.device
            v = draft.spec.vocab
            self.markov = tuple((torch.randn(v, MARKOV_RANK, generator=g) * 0.05).to(torch.bfloat16).to(dev) for _ in range(2))

    def _markov_children_fn(self, ds):
        """One greedy draft chain gives a base-logit row per depth; children come from the Markov head."""
        from ..ops import markov_ops
        de = self.draft.engine
        w1, w2 = self.markov
        chain, base = [ds.pending_token], []

        def base_row(depth: int) -> None:
            while len(base) <= depth:
                lg = de.forward_rows(ds, chain, return_logits=True)[-1]
                self.draft_forwards += 1
                base.append(lg.to(torch.bfloat16))
                chain.append(int(torch.argmax(lg.float())))

        def fn(paths: list[list[int]]):
            depths = [min(len(p) - 1, MARKOV_DEPTH - 1) for p in paths]
            base_row(max(depths))
            dev = w1.device
            top4, logp, _ = markov_ops.markov_top4(w1, w2, torch.stack(base).contiguous(),
                                                   torch.tensor([p[-1] for p in paths], dtype=torch.int32, device=dev),
                                                   torch.tensor(depths, dtype=torch.int32, device=dev))
            t, l = top4.cpu().tolist(), logp.cpu().tolist()
            return [list(zip(a, b)) for a, b in zip(t, l)]
        return fn

    def _children_fn(self, ds):
        de = self.draft.engine

        def fn(paths: list[list[int]]):
            outs = []
            for p in paths:
                logits = de.forward_rows(ds, p, return_logits=True)[-1].float()
                self.draft_forwards += 1
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
                if self.builder == "markov":
                    ds.pending_token = ts.pending
                    tree = build_tree(ts.pending, self._markov_children_fn(ds), self.rows, "waves")
                else:
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
