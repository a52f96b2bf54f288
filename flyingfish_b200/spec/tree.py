"""Draft trees for speculative decoding.

A tree has at most 64 rows (``tree16 / tree32 / tree64`` budgets) and depth at most 7; row 0 is the
root (the pending token). Nodes are added best-first by cumulative path log-probability with
deterministic ties (lower parent row, then lower child rank), each node carries its ancestor set as
a 64-bit mask (bit i = row i is an ancestor-or-self) which is exactly what the verification
attention kernel consumes as its per-row visibility mask (``attn_decode(tree_mask=...)``). The
``waves`` builder expands level by level from batched top-k distributions (one draft forward per
level), ``serial`` expands one node at a time. Mirrors the reference's tree machinery
(src/tree.rs:7-160, 213-430; budgets src/backend/mod.rs:100-166).
"""
from __future__ import annotations

import heapq
import math
from dataclasses import dataclass, field
from typing import Callable

BUDGETS = {"chain": 0, "tree16": 16, "tree32": 32, "tree64": 64}
MAX_DEPTH = 7
TOP_CHILDREN = 4


@dataclass
class Tree:
    tokens: list[int] = field(default_factory=list)        # token of each row (row 0 = pending token)
    parents: list[int] = field(default_factory=list)       # parent row (-1 for the root)
    depth: list[int] = field(default_factory=list)
    logp: list[float] = field(default_factory=list)        # cumulative path log-probability
    masks: list[int] = field(default_factory=list)         # ancestor-or-self bit sets

    def add(self, token: int, parent: int, logp: float) -> int:
        row = len(self.tokens)
        assert row < 64, "a verification tree holds at most 64 rows"
        self.tokens.append(token)
        self.parents.append(parent)
        self.depth.append(0 if parent < 0 else self.depth[parent] + 1)
        self.logp.append(logp)
        self.masks.append((1 << row) | (self.masks[parent] if parent >= 0 else 0))
        return row

    def __len__(self) -> int:
        return len(self.tokens)

    def positions(self, base: int) -> list[int]:
        """Sequence position of every row when the root sits at position ``base``."""
        return [base + d for d in self.depth]

    def path(self, row: int) -> list[int]:
        out = []
        while row >= 0:
            out.append(row)
            row = self.parents[row]
        return out[::-1]

    def check(self) -> None:
        for r in range(len(self)):
            p = self.parents[r]
            assert (p == -1) == (r == 0) and p < r, "parents must precede children"
            assert self.masks[r] & ((1 << (r + 1)) - 1) == self.masks[r], "mask may only name earlier rows"
            assert self.depth[r] <= MAX_DEPTH


# children_fn(node_tokens_path) -> list of (token, logprob) sorted by decreasing probability
ChildrenFn = Callable[[list[list[int]]], list[list[tuple[int, float]]]]


def build_tree(root_token: int, children_fn: ChildrenFn, budget: int, builder: str = "waves",
               max_depth: int = MAX_DEPTH, top_children: int = TOP_CHILDREN) -> Tree:
    """Best-first tree of ``budget`` rows. ``children_fn`` receives a batch of token paths (from the
    root) and returns the draft model's top candidates for the next token of each path."""
    t = Tree()
    t.add(root_token, -1, 0.0)
    if budget <= 1:
        return t
    # heap of candidate nodes: (-logp, parent_row, rank, token)
    heap: list[tuple[float, int, int, int]] = []

    def expand(rows: list[int]) -> None:
        paths = [[t.tokens[r] for r in t.path(r_)] for r_ in rows for r in [r_]]
        outs = children_fn(paths)
        for r, cands in zip(rows, outs):
            if t.depth[r] >= max_depth:
                continue
            for rank, (tok, lp) in enumerate(cands[:top_children]):
                heapq.heappush(heap, (-(t.logp[r] + lp), r, rank, tok))

    if builder == "serial":
        expand([0])
        while heap and len(t) < budget:
            nlp, parent, rank, tok = heapq.heappop(heap)
            row = t.add(tok, parent, -nlp)
            if len(t) < budget:
                expand([row])
    else:
        frontier = [0]
        while frontier and len(t) < budget:
            expand(frontier)
            frontier = []
            # take the best candidates of this wave: at most what the budget allows, and never a
            # candidate worse than one left in the heap from an earlier wave
            take = min(budget - len(t), max(1, len(heap)))
            wave: list[int] = []
            for _ in range(take):
                if not heap:
                    break
                nlp, parent, rank, tok = heapq.heappop(heap)
                wave.append(t.add(tok, parent, -nlp))
            frontier = [r for r in wave if t.depth[r] < max_depth]
    t.check()
    return t


@dataclass
class VerifyCostSchedule:
    """MoE-aware verification width (src/dspark.rs:107-340, 897-930): more rows touch more experts,
    so a draft position is only verified while its cumulative confidence stays above ``tau`` and the
    expected gain beats the expected expert-fetch cost. Rows are clamped to [2, 8]."""
    tau: float = 0.80
    min_rows: int = 2
    max_rows: int = 8
    miss_cost_ms: float = 0.0            # cost of fetching one non-resident expert
    step_ms: float = 1.0                 # cost of one plain decode step
    expected_new_experts_per_row: float = 0.0

    def survival_floor(self) -> float:
        """Minimum survival probability at which verifying one more row pays for itself."""
        extra = self.miss_cost_ms * self.expected_new_experts_per_row
        return min(0.99, extra / max(self.step_ms, 1e-9))

    def select_rows(self, confidences: list[float]) -> int:
        """``confidences[j]`` = draft probability of token j given the previous ones. Returns the
        number of rows (pending token included) to verify."""
        rows, surv = 1, 1.0
        floor = self.survival_floor()
        for c in confidences:
            surv *= c
            if rows >= self.min_rows and (c < self.tau and surv < max(floor, 1e-9) or surv < floor):
                break
            rows += 1
            if rows >= self.max_rows:
                break
        return max(self.min_rows, min(rows, self.max_rows, len(confidences) + 1))
