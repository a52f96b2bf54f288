"""Leader / follower execution of one engine over several ranks.

A tensor- or expert-parallel model needs every rank to issue the same sequence of engine calls:
the kernels of a step meet each other through peer memory and collectives. ``generate`` and
``bench`` are deterministic programs, so every rank simply runs them (SPMD). A server is not: only
rank 0 sees the requests. ``EngineLeader`` wraps rank 0's engine; every state-changing call is
first broadcast as a small descriptor ``(method, args)`` over a host-side (gloo) group and then
executed locally, and the other ranks sit in :func:`follow`, executing the same calls on their own
engine until the leader says stop. The descriptor carries only host data (token ids, sequence ids,
chunk size), never tensors.

The reference has no counterpart (one process, one device: src/serve/mod.rs:179-218); this is the
distributed form of its engine thread.
"""
from __future__ import annotations

from typing import Any

import torch.distributed as dist

STOP = "__stop__"
_FORWARDED = ("add_sequence", "free_sequence", "prefill", "prefill_some", "decode", "reset", "capture")


def _bcast(group, obj: Any, src: int = 0) -> Any:
    box = [obj]
    dist.broadcast_object_list(box, src=src, group=group)
    return box[0]


class EngineLeader:
    """Rank 0's engine, with every forwarded call announced to the followers first. Sequences are named by id on
    the wire; both sides create them in the same order, so the ids agree."""

    def __init__(self, engine, group):
        self._engine, self._group = engine, group

    def __getattr__(self, name):
        attr = getattr(self._engine, name)
        if name not in _FORWARDED:
            return attr

        def call(*args, **kw):
            wire_args = [self._wire(a) for a in args]
            wire_kw = {k: self._wire(v) for k, v in kw.items()}
            _bcast(self._group, (name, wire_args, wire_kw))
            return attr(*args, **kw)
        return call

    def __setattr__(self, name, value):
        if name.startswith("_"):
            object.__setattr__(self, name, value)
        else:
            setattr(self._engine, name, value)

    @staticmethod
    def _wire(a):
        if isinstance(a, list) and a and hasattr(a[0], "seq_id"):
            return ("seqs", [s.seq_id for s in a])
        if hasattr(a, "seq_id"):
            return ("seq", a.seq_id)
        return ("val", a)

    def stop(self) -> None:
        _bcast(self._group, (STOP, [], {}))


def follow(engine, group) -> int:
    """Run on every rank but the leader: execute the leader's calls until it stops. Returns the number of calls
    executed. A failing call poisons the local engine (as it does on the leader) and ends the loop by raising."""
    n = 0

    def unwire(a):
        kind, v = a
        if kind == "seqs":
            return [engine.seqs[i] for i in v]
        if kind == "seq":
            return engine.seqs[v]
        return v
    while True:
        name, args, kw = _bcast(group, None)
        if name == STOP:
            return n
        getattr(engine, name)(*[unwire(a) for a in args], **{k: unwire(v) for k, v in kw.items()})
        n += 1
