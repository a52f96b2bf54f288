"""Engine thread and admission for the server.

One thread owns the engine (and every CUDA handle); HTTP handlers talk to it through a command
queue and receive ``EngineEvent``s through per-request asyncio queues -- the same split as the
reference (engine thread + channels, src/serve/mod.rs:20-39, 179-259). Differences that follow
from continuous batching: admission is a bounded number of in-flight requests instead of a
single slot (the reference answers 409 while one request runs, src/serve/mod.rs:41-102), and an
aborted request only frees its own sequence.

Failure policy is the reference's: an exception escaping a scheduler iteration fails every
in-flight request, marks the backend ``unavailable`` for good and ends the loop
(src/serve/mod.rs:261-289).
"""
from __future__ import annotations

import asyncio
import queue
import threading
import time
import traceback
from dataclasses import dataclass, field

from ..engine.scheduler import Request, Scheduler
from ..utils.log import log_json


@dataclass
class EngineEvent:
    kind: str                      # tokens | done | aborted | failed
    tokens: list[int] = field(default_factory=list)
    finish_reason: str | None = None
    message: str | None = None


class Busy(RuntimeError):
    pass


class Unavailable(RuntimeError):
    pass


class Backend:
    """Thread-safe front of the engine thread."""

    def __init__(self, engine, eos_ids: tuple[int, ...] = (), max_inflight: int | None = None,
                 token_budget: int | None = None):
        self.engine = engine
        self.scheduler = Scheduler(engine, token_budget=token_budget)
        self.eos_ids = eos_ids
        self.max_inflight = max_inflight or 4 * engine.max_batch
        self.state = "idle"            # idle | running | unavailable
        self._cmd: queue.Queue = queue.Queue()
        self._inflight: dict[int, tuple[Request, asyncio.Queue, asyncio.AbstractEventLoop]] = {}
        self._lock = threading.Lock()
        self._thread = threading.Thread(target=self._loop, name="engine", daemon=True)
        self._stop = False
        self.served = 0
        self.ttft_ms: list[float] = []

    def start(self) -> None:
        self._thread.start()

    def shutdown(self) -> None:
        self._stop = True
        self._cmd.put(("stop", None))
        self._thread.join(timeout=10)

    # -- called from the event loop thread --------------------------------------------------
    def add_request(self, prompt: list[int], max_tokens: int, ignore_eos: bool = False,
                    images: list | None = None) -> tuple[Request, asyncio.Queue]:
        if self.state == "unavailable":
            raise Unavailable("engine is unavailable after an earlier failure")
        with self._lock:
            if len(self._inflight) >= self.max_inflight:
                raise Busy("busy: too many requests in flight")
            loop = asyncio.get_running_loop()
            q: asyncio.Queue = asyncio.Queue()
            req = Request(prompt=prompt, max_tokens=max_tokens, eos_ids=self.eos_ids, ignore_eos=ignore_eos,
                          images=images or None)
            req.on_tokens = self._on_tokens
            req.on_finish = self._on_finish
            self._inflight[req.req_id] = (req, q, loop)
        self._cmd.put(("add", req))
        return req, q

    def abort(self, req: Request) -> None:
        self._cmd.put(("abort", req))

    # -- engine thread -----------------------------------------------------------------------
    def _post(self, req: Request, ev: EngineEvent) -> None:
        ent = self._inflight.get(req.req_id)
        if ent is None:
            return
        _, q, loop = ent
        loop.call_soon_threadsafe(q.put_nowait, ev)

    def _on_tokens(self, req: Request, toks: list[int]) -> None:
        self._post(req, EngineEvent("tokens", tokens=list(toks)))

    def _on_finish(self, req: Request) -> None:
        kind = "aborted" if req.state == "aborted" else "done"
        self._post(req, EngineEvent(kind, finish_reason=req.finish_reason))
        if req.ttft_ms is not None:
            self.ttft_ms.append(req.ttft_ms)
        log_json("serve_request", verbose_only=True, req=req.req_id, prompt_tokens=len(req.prompt),
                 completion_tokens=len(req.output), finish=req.finish_reason, ttft_ms=req.ttft_ms)
        with self._lock:
            self._inflight.pop(req.req_id, None)
        self.served += 1

    def _drain_commands(self, block: bool) -> None:
        while True:
            try:
                cmd, arg = self._cmd.get(block=block, timeout=0.05 if block else None)
            except queue.Empty:
                return
            block = False
            if cmd == "add":
                try:
                    self.scheduler.submit(arg)
                except Exception as e:  # rejected before scheduling (capacity)
                    arg.state, arg.finish_reason, arg.error = "failed", None, str(e)
                    self._post(arg, EngineEvent("failed", message=str(e)))
                    with self._lock:
                        self._inflight.pop(arg.req_id, None)
            elif cmd == "abort":
                self.scheduler.abort(arg)
            elif cmd == "stop":
                return

    def _loop(self) -> None:
        try:
            while not self._stop:
                self._drain_commands(block=not self.scheduler.has_work())
                if self._stop:
                    break
                if self.scheduler.has_work():
                    self.state = "running"
                    self.scheduler.step()
                else:
                    self.state = "idle"
        except Exception as e:  # engine failure: fail everything, become unavailable
            self.state = "unavailable"
            msg = f"{type(e).__name__}: {e}"
            log_json("engine_failure", error=msg, trace=traceback.format_exc()[-2000:])
            with self._lock:
                items = list(self._inflight.values())
                self._inflight.clear()
            for req, q, loop in items:
                req.state = "failed"
                loop.call_soon_threadsafe(q.put_nowait, EngineEvent("failed", message=msg))

    def p50_ttft_ms(self) -> float | None:
        if not self.ttft_ms:
            return None
        s = sorted(self.ttft_ms)
        return s[len(s) // 2]


class MtpBackend(Backend):
    """Server backend for ``ff serve --mtp N``: every request is generated by multi-token-prediction speculation
    (draft with the MTP head, verify with one multi-row target forward). Speculation rounds are per sequence, so
    admission is the reference's single slot (src/serve/mod.rs:41-59, ``run_mtp`` :144-161): a second request while
    one runs is answered 409."""

    def __init__(self, model, depth: int, eos_ids: tuple[int, ...] = ()):
        super().__init__(model.engine, eos_ids=eos_ids, max_inflight=1)
        from ..spec.mtp import MtpSpeculator
        self.spec = MtpSpeculator(model, depth=depth)
        self.depth = depth

    def _loop(self) -> None:
        try:
            while not self._stop:
                try:
                    cmd, req = self._cmd.get(timeout=0.05)
                except queue.Empty:
                    self.state = "idle"
                    continue
                if cmd == "stop":
                    break
                if cmd == "abort":
                    req.state = "aborted"
                    continue
                if cmd != "add" or req.state == "aborted":
                    continue
                self.state = "running"
                req.state = "running"

                def on_tokens(toks, req=req):
                    if req.first_token_time is None:
                        req.first_token_time = time.perf_counter()
                    req.output.extend(toks)
                    self._on_tokens(req, toks)

                def should_stop(req=req):
                    # an abort for this request may be waiting in the queue
                    try:
                        while True:
                            c, r = self._cmd.get_nowait()
                            if c == "abort" and r is req:
                                req.state = "aborted"
                            elif c == "stop":
                                self._stop = True
                                req.state = "aborted"
                            else:
                                self._cmd.put((c, r))
                                break
                    except queue.Empty:
                        pass
                    return req.state == "aborted"

                if len(req.prompt) + req.max_tokens + self.depth + 1 > self.engine.settings.capacity:
                    req.state, req.error = "failed", "prompt + max_tokens exceeds the KV capacity"
                    self._post(req, EngineEvent("failed", message=req.error))
                    with self._lock:
                        self._inflight.pop(req.req_id, None)
                    continue
                out = self.spec.generate(req.prompt, req.max_tokens, ignore_eos=req.ignore_eos, on_tokens=on_tokens,
                                         should_stop=should_stop)
                if req.state == "aborted":
                    req.finish_reason = "aborted"
                else:
                    last = out.ids[-1] if out.ids else None
                    req.state = "finished"
                    req.finish_reason = "stop" if (not req.ignore_eos and last in self.eos_ids) else "length"
                self._on_finish(req)
        except Exception as e:
            self.state = "unavailable"
            msg = f"{type(e).__name__}: {e}"
            log_json("engine_failure", error=msg, trace=traceback.format_exc()[-2000:])
            with self._lock:
                items = list(self._inflight.values())
                self._inflight.clear()
            for req, q, loop in items:
                req.state = "failed"
                loop.call_soon_threadsafe(q.put_nowait, EngineEvent("failed", message=msg))
