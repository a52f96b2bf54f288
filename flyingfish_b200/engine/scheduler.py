"""Continuous-batching scheduler.

The reference serves one request at a time through a single admission slot
(src/serve/mod.rs:41-59; busy -> HTTP 409). A 180 GB part with a paged cache can hold hundreds of
sequences, so this build schedules many. Every iteration has a token budget shared by the decode
batch and ONE packed prefill chunk: waiting requests are admitted while KV blocks and batch slots
are free, every sequence that is already generating decodes one token, and the rest of the budget
goes to prompt rows of the sequences still prefilling (oldest first). A long prompt is therefore
spread over several iterations and never stalls the running streams for more than one chunk.
Requests can be aborted at any iteration (client disconnect), which frees their blocks at once.

The scheduler is synchronous and engine-agnostic (it only needs ``add_sequence / prefill /
decode / free_sequence``), so its policy is unit-tested on CPU with a scripted fake engine.
"""
from __future__ import annotations

import itertools
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable

from .kv_cache import OutOfBlocks


@dataclass
class Request:
    prompt: list[int]
    max_tokens: int
    eos_ids: tuple[int, ...] = ()
    ignore_eos: bool = False
    on_tokens: Callable[["Request", list[int]], None] | None = None     # streaming callback
    on_finish: Callable[["Request"], None] | None = None
    req_id: int = field(default_factory=itertools.count().__next__)
    state: str = "waiting"            # waiting | running | finished | aborted | failed
    finish_reason: str | None = None  # stop | length | aborted
    output: list[int] = field(default_factory=list)
    seq: object | None = None
    arrival: float = field(default_factory=time.perf_counter)
    first_token_time: float | None = None
    error: str | None = None
    images: list | None = None        # decoded images, one per image placeholder token of ``prompt``
    mm_positions: list[int] | None = None
    mm_embeds: object | None = None

    @property
    def ttft_ms(self) -> float | None:
        return None if self.first_token_time is None else (self.first_token_time - self.arrival) * 1e3


class Scheduler:
    def __init__(self, engine, max_running: int | None = None, prefill_chunk: int | None = None,
                 token_budget: int | None = None):
        self.engine = engine
        self.max_running = max_running or engine.max_batch
        self.prefill_chunk = prefill_chunk
        # rows one iteration may process: decode rows first, the remainder is the prefill chunk
        self.token_budget = token_budget or prefill_chunk or getattr(engine, "max_prefill_rows", 8192)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []
        self.stats = {"admitted": 0, "finished": 0, "aborted": 0, "iterations": 0, "preempted": 0}

    # -- API -----------------------------------------------------------------------------------
    def submit(self, req: Request) -> Request:
        if req.images and req.mm_positions is None:
            # runs on the engine thread: vision tower over the images, placeholders expanded to their spans
            enc = getattr(self.engine, "mm_encoder", None)
            if enc is None:
                raise ValueError("this model has no vision tower: image input is not supported")
            req.prompt, req.mm_positions, req.mm_embeds = enc(req.prompt, req.images)
        if len(req.prompt) + req.max_tokens > self.engine.settings.capacity:
            raise ValueError(f"prompt ({len(req.prompt)}) + max_tokens ({req.max_tokens}) exceeds the KV capacity "
                             f"{self.engine.settings.capacity}")
        self.waiting.append(req)
        return req

    def abort(self, req: Request) -> None:
        if req.state in ("finished", "aborted", "failed"):
            return
        if req.state == "running":
            self.running.remove(req)
            self.engine.free_sequence(req.seq.seq_id)
        else:
            try:
                self.waiting.remove(req)
            except ValueError:
                pass
        req.state, req.finish_reason = "aborted", "aborted"
        self.stats["aborted"] += 1
        if req.on_finish:
            req.on_finish(req)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # -- one iteration -------------------------------------------------------------------------
    def _blocks_for(self, tokens: int) -> int:
        bs = self.engine.kv.block_size
        return (tokens + bs - 1) // bs

    def _admit(self) -> list[Request]:
        admitted = []
        free = self.engine.kv.alloc.free_blocks
        # blocks already promised to running sequences for their remaining growth are not
        # reserved: a sequence that cannot grow is preempted (see _decode)
        while self.waiting and len(self.running) + len(admitted) < self.max_running:
            req = self.waiting[0]
            need = self._blocks_for(len(req.prompt) + len(req.output) + 1)
            if need > free:
                break
            free -= need
            self.waiting.popleft()
            # a preempted request resumes by recomputing prompt + what it already produced
            if req.mm_positions:
                req.seq = self.engine.add_sequence(req.prompt + req.output, req.mm_positions, req.mm_embeds)
            else:
                req.seq = self.engine.add_sequence(req.prompt + req.output)
            req.state = "running"
            admitted.append(req)
            self.stats["admitted"] += 1
        return admitted

    def _emit(self, req: Request, toks: list[int]) -> None:
        if req.first_token_time is None:
            req.first_token_time = time.perf_counter()
        req.output.extend(toks)
        if req.on_tokens:
            req.on_tokens(req, toks)

    def _maybe_finish(self, req: Request) -> bool:
        last = req.output[-1] if req.output else None
        reason = None
        if not req.ignore_eos and last is not None and last in req.eos_ids:
            reason = "stop"
        elif len(req.output) >= req.max_tokens:
            reason = "length"
        if reason is None:
            return False
        req.state, req.finish_reason = "finished", reason
        self.engine.free_sequence(req.seq.seq_id)
        self.stats["finished"] += 1
        if req.on_finish:
            req.on_finish(req)
        return True

    def _preempt_youngest(self) -> None:
        """Out of KV blocks: the youngest running request goes back to the queue (it will be recomputed from its
        prompt plus what it already produced)."""
        victim = self.running.pop()
        self.engine.free_sequence(victim.seq.seq_id)
        victim.state, victim.seq = "waiting", None
        self.waiting.appendleft(victim)
        self.stats["preempted"] += 1

    def step(self) -> int:
        """Run one scheduling iteration; returns the number of tokens produced."""
        self.stats["iterations"] += 1
        produced = 0
        self.running.extend(self._admit())
        decoding = [r for r in self.running if r.seq.prefilled >= len(r.seq.prompt)][: self.engine.max_batch]
        prefilling = [r for r in self.running if r.seq.prefilled < len(r.seq.prompt)]
        # ---- decode step of every generating sequence ----
        if decoding:
            try:
                toks = self.engine.decode([r.seq for r in decoding])
            except OutOfBlocks:
                self._preempt_youngest()
                return 0
            for r, t in zip(decoding, toks):
                self._emit(r, [t])
                produced += 1
        # ---- one prefill chunk with what is left of the budget ----
        rows = self.token_budget - len(decoding)
        if prefilling and rows > 0:
            try:
                done = self.engine.prefill_some([r.seq for r in prefilling], rows)
            except OutOfBlocks:
                self._preempt_youngest()
                return produced
            finished_ids = {s.seq_id for s in done}
            for r in prefilling:
                if r.seq.seq_id in finished_ids:
                    self._emit(r, [r.seq.output[-1]])
                    produced += 1
        self.running = [r for r in self.running if r.state == "running" and not (r.output and self._maybe_finish(r))]
        return produced

    def run_until_idle(self, max_iters: int = 1_000_000) -> None:
        it = 0
        while self.has_work() and it < max_iters:
            self.step()
            it += 1
