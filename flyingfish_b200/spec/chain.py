"""Chain speculation with a draft model: draft k tokens autoregressively with a small model,
verify them with ONE multi-row forward of the target, accept the matching prefix plus the
target's bonus token, roll the draft model's cache back to the accepted length.

Transactional like the reference's rounds (src/mtp/transaction.rs:18-155: save checkpoint ->
draft -> verify -> restore -> publish): both caches only ever *commit* accepted rows, so a
failure at any stage leaves the committed state untouched; the host-side ``Fault`` enum injects
failures at each stage for the tests (src/mtp/transaction.rs:5-14).
"""
from __future__ import annotations

import enum
import time
from dataclasses import dataclass, field

from ..api import GenerationOutput, Model
from .accept import accept_chain


class Fault(enum.Enum):
    NONE = 0
    DRAFT = 1
    VERIFY = 2
    COMMIT = 3


class SpecFault(RuntimeError):
    pass


@dataclass
class SpecStats:
    rounds: int = 0
    drafted: int = 0
    accepted: int = 0
    emitted: int = 0
    accepted_per_round: list[int] = field(default_factory=list)

    @property
    def acceptance_rate(self) -> float:
        return self.accepted / self.drafted if self.drafted else 0.0

    @property
    def tokens_per_round(self) -> float:
        return self.emitted / self.rounds if self.rounds else 0.0


class ChainSpeculator:
    """Target + draft model pair bound to one sequence each."""

    def __init__(self, target: Model, draft: Model, k: int = 4):
        assert target.spec.vocab == draft.spec.vocab, "draft and target must share a vocabulary"
        self.target, self.draft, self.k = target, draft, k
        self.stats = SpecStats()
        self.fault = Fault.NONE

    def generate(self, ids: list[int], count: int, ignore_eos: bool = True) -> GenerationOutput:
        te, de = self.target.engine, self.draft.engine
        eos = tuple(self.target.spec.extra.get("eos_token_ids", [self.target.spec.eos_token_id]
                                                if self.target.spec.eos_token_id is not None else []))
        if len(ids) + count + self.k + 1 > te.settings.capacity:
            raise ValueError("prompt + output + draft rows exceed the KV capacity")
        t0 = time.perf_counter()
        ts = te.add_sequence(ids)
        ds = de.add_sequence(ids)
        try:
            first = te.prefill([ts])[0]
            de.prefill([ds])
            # the draft model's own first token is discarded: it continues from the target's
            ds.output.clear()
            ds.pending = first
            out = [first]
            t1 = time.perf_counter()
            while len(out) < count and not (not ignore_eos and eos and out[-1] in eos):
                k = min(self.k, count - len(out))
                emitted = self._round(ts, ds, k, eos, ignore_eos)
                out.extend(emitted)
            out = out[:count]
            t2 = time.perf_counter()
            return GenerationOutput(ids=out, prefill_ms=(t1 - t0) * 1e3, decode_ms=(t2 - t1) * 1e3,
                                    decode_steps=self.stats.rounds,
                                    extra={"accepted_per_round": self.stats.accepted_per_round,
                                           "acceptance_rate": self.stats.acceptance_rate})
        finally:
            te.free_sequence(ts.seq_id)
            de.free_sequence(ds.seq_id)

    def _round(self, ts, ds, k: int, eos, ignore_eos: bool) -> list[int]:
        te, de = self.target.engine, self.draft.engine
        base_len = de.kv.seqs[ds.seq_id].length
        # ---- draft ----
        if self.fault is Fault.DRAFT:
            raise SpecFault("injected draft failure")
        drafts: list[int] = []
        for _ in range(k):
            drafts.append(de.decode([ds])[0])
        # ---- verify ----
        if self.fault is Fault.VERIFY:
            de.kv.truncate(ds.seq_id, base_len)
            raise SpecFault("injected verify failure")
        target_toks = te.verify([ts], [drafts])[0]
        acc = accept_chain(drafts, target_toks, eos, ignore_eos)
        # ---- commit ----
        if self.fault is Fault.COMMIT:
            de.kv.truncate(ds.seq_id, base_len)
            raise SpecFault("injected commit failure")
        te.commit_verified(ts, acc.tokens, acc.n_draft_accepted)
        # draft cache: it holds rows for the pending token and drafts 1..k-1; keep the pending
        # token's row and the accepted drafts' rows
        if acc.n_draft_accepted == k:
            # every draft matched: the draft model has not consumed its own last token yet
            ds.pending = drafts[-1]
            de.decode([ds])                 # fills the KV row of the last accepted draft
        else:
            de.kv.truncate(ds.seq_id, base_len + acc.n_draft_accepted + 1)
        ds.output.clear()
        ds.pending = acc.tokens[-1]
        st = self.stats
        st.rounds += 1; st.drafted += k; st.accepted += acc.n_draft_accepted; st.emitted += len(acc.tokens)
        st.accepted_per_round.append(acc.n_draft_accepted)
        return acc.tokens
