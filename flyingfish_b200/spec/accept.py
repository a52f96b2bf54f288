"""Greedy acceptance for speculative decoding.

Accept the longest prefix where the draft token equals the target's argmax, then append the
target's own token at the first mismatch (the "bonus" token); an EOS inside the accepted prefix
truncates the emission. The emitted stream is therefore identical to plain greedy decoding
(the reference's ``accept``, src/dspark.rs:932-950; batched MTP, src/mtp/batched.rs:135-146).
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class Accepted:
    tokens: list[int]        # tokens to emit this round (accepted drafts + bonus)
    n_draft_accepted: int    # how many draft tokens matched
    hit_eos: bool = False


def accept_chain(draft: list[int], target: list[int], eos_ids: tuple[int, ...] = (), ignore_eos: bool = True) -> Accepted:
    """``target[j]`` is the target model's greedy token after consuming the pending token and
    ``draft[:j]``; ``len(target) == len(draft) + 1``."""
    assert len(target) == len(draft) + 1
    out: list[int] = []
    n = 0
    for j, d in enumerate(draft):
        if d != target[j]:
            break
        out.append(d)
        n += 1
        if not ignore_eos and d in eos_ids:
            return Accepted(out, n, True)
    out.append(target[n])
    hit = (not ignore_eos) and out[-1] in eos_ids
    return Accepted(out, n, hit)


def accept_tree(parents: list[int], tokens: list[int], target: list[int], eos_ids: tuple[int, ...] = (),
                ignore_eos: bool = True) -> tuple[Accepted, list[int]]:
    """Tree variant: node 0 is the root (the pending token); ``tokens[i]`` is the draft token of
    node i (i >= 1), ``parents[i]`` its parent, ``target[i]`` the target's greedy token after the
    path ending in node i. Walks from the root, at every node following the child whose token
    equals the target's prediction (lowest node index on duplicates). Returns the emission and
    the accepted node path (root first)."""
    children: dict[int, list[int]] = {}
    for i in range(1, len(parents)):
        children.setdefault(parents[i], []).append(i)
    path = [0]
    out: list[int] = []
    cur = 0
    while True:
        want = target[cur]
        nxt = next((c for c in children.get(cur, []) if tokens[c] == want), None)
        if nxt is None:
            out.append(want)
            break
        out.append(tokens[nxt])
        path.append(nxt)
        cur = nxt
        if not ignore_eos and tokens[nxt] in eos_ids:
            return Accepted(out, len(path) - 1, True), path
    hit = (not ignore_eos) and out[-1] in eos_ids
    return Accepted(out, len(path) - 1, hit), path
