"""Continuous-batching scheduler: token budget shared by the decode batch and one prefill chunk per iteration,
admission by free KV blocks, preemption, abort. Policy tests run against a scripted engine; the interleaving test runs
the real engine on CPU and checks the tokens against unscheduled generation."""
import asyncio

import pytest

from flyingfish_b200.engine.kv_cache import OutOfBlocks
from flyingfish_b200.engine.scheduler import Request, Scheduler


class _Alloc:
    def __init__(self, n):
        self.free_blocks = n


class _KV:
    def __init__(self, blocks, block_size=16):
        self.alloc, self.block_size = _Alloc(blocks), block_size


class _Settings:
    capacity = 4096


class _Seq:
    def __init__(self, sid, prompt):
        self.seq_id, self.prompt, self.output, self.prefilled, self.pending = sid, list(prompt), [], 0, None


class FakeEngine:
    """Token i of a sequence is 1000 * seq_id + i; records every call with its row count."""
    max_batch, max_prefill_rows, settings = 4, 64, _Settings()

    def __init__(self, blocks=1000):
        self.kv = _KV(blocks)
        self.seqs, self.calls, self._next = {}, [], 0
        self.fail_decode_with_oob = 0

    def add_sequence(self, prompt, *a):
        s = _Seq(self._next, prompt); self._next += 1
        self.seqs[s.seq_id] = s
        self.kv.alloc.free_blocks -= (len(prompt) + 1 + 15) // 16
        return s

    def free_sequence(self, sid):
        s = self.seqs.pop(sid)
        self.kv.alloc.free_blocks += (len(s.prompt) + 1 + 15) // 16

    def prefill_some(self, seqs, max_rows):
        left, done, rows = max_rows, [], 0
        for s in seqs:
            take = min(len(s.prompt) - s.prefilled, left)
            if take <= 0:
                continue
            s.prefilled += take; left -= take; rows += take
            if s.prefilled == len(s.prompt):
                s.output.append(1000 * s.seq_id); s.pending = s.output[-1]
                done.append(s)
        self.calls.append(("prefill", rows))
        return done

    def decode(self, seqs):
        if self.fail_decode_with_oob:
            self.fail_decode_with_oob -= 1
            raise OutOfBlocks("scripted")
        self.calls.append(("decode", len(seqs)))
        out = []
        for s in seqs:
            s.output.append(1000 * s.seq_id + len(s.output)); s.pending = s.output[-1]
            out.append(s.output[-1])
        return out


def test_budget_is_shared_by_decode_rows_and_one_prefill_chunk():
    eng = FakeEngine()
    sch = Scheduler(eng, token_budget=32)
    short = Request(prompt=list(range(10)), max_tokens=6, ignore_eos=True)
    sch.submit(short)
    sch.step()                                     # the short prompt fits one chunk: first token out
    assert short.output == [0] and eng.calls == [("prefill", 10)]
    long = Request(prompt=list(range(100)), max_tokens=3, ignore_eos=True)
    sch.submit(long)
    trace = []
    while long.state != "finished" or short.state != "finished":
        before = len(short.output)
        sch.step()
        trace.append((len(short.output) - before, long.seq.prefilled if long.seq else None))
    # while the long prompt was prefilled chunk by chunk (31 rows per iteration: the budget minus the decode row), the
    # short request produced a token in every iteration
    chunks = [c for c in eng.calls if c[0] == "prefill"][1:]
    assert [r for _, r in chunks][:3] == [31, 31, 31] and sum(r for _, r in chunks) == 100
    assert all(d == 1 for d, _ in trace[:4])
    assert short.output == [0, 1, 2, 3, 4, 5] and long.output == [1000, 1001, 1002]


def test_admission_waits_for_blocks_and_slots():
    eng = FakeEngine(blocks=5)                     # 16-token blocks: a 40-token prompt needs 3
    sch = Scheduler(eng, token_budget=64)
    a, b = (Request(prompt=list(range(40)), max_tokens=2, ignore_eos=True) for _ in range(2))
    sch.submit(a); sch.submit(b)
    sch.step()
    assert a.state == "running" and b.state == "waiting"          # only one fits
    sch.run_until_idle()
    assert a.state == b.state == "finished" and sch.stats["admitted"] == 2


def test_out_of_blocks_preempts_the_youngest_and_recomputes_it():
    eng = FakeEngine()
    sch = Scheduler(eng, token_budget=64)
    a = Request(prompt=list(range(8)), max_tokens=4, ignore_eos=True)
    b = Request(prompt=list(range(8)), max_tokens=4, ignore_eos=True)
    sch.submit(a); sch.submit(b)
    sch.step()
    eng.fail_decode_with_oob = 1
    assert sch.step() == 0 and sch.stats["preempted"] == 1 and b.state == "waiting" and b.seq is None
    sch.run_until_idle()
    assert a.state == b.state == "finished" and len(b.output) == 4


def test_abort_frees_the_sequence():
    eng = FakeEngine()
    sch = Scheduler(eng, token_budget=16)
    r = Request(prompt=list(range(40)), max_tokens=4, ignore_eos=True)
    sch.submit(r)
    sch.step()
    free = eng.kv.alloc.free_blocks
    sch.abort(r)
    assert r.state == "aborted" and eng.kv.alloc.free_blocks > free and not sch.has_work()


def test_real_engine_interleaves_and_matches_plain_generation():
    """CPU engine, budget of 24 rows: a 90-token prompt arrives while another request decodes. The decoding request
    keeps emitting between the chunks of the long prefill, and both requests produce exactly the tokens of running
    them alone (chunked prefill and batching do not change results)."""
    from flyingfish_b200.api import Model, generate_plain
    from flyingfish_b200.config import Settings
    from flyingfish_b200.serve.backend import Backend
    m = Model.load("tiny-llama", Settings(capacity=256, max_batch=4, graph=False), device="cpu", seed=0)
    pa, pb = list(range(5, 25)), [(7 * i) % 2000 + 3 for i in range(90)]
    alone = []
    for p, n in ((pa, 12), (pb, 4)):
        alone.append(generate_plain(m, p, n, ignore_eos=True, graph=False).ids)
        m.reset()

    async def main():
        be = Backend(m.engine, eos_ids=(), token_budget=24)
        be.start()
        try:
            ra, qa = be.add_request(pa, 12, ignore_eos=True)
            first = await asyncio.wait_for(qa.get(), timeout=60)
            assert first.kind == "tokens"
            rb, qb = be.add_request(pb, 4, ignore_eos=True)
            order = []
            done = set()
            async def drain(tag, q):
                toks = []
                while True:
                    ev = await asyncio.wait_for(q.get(), timeout=120)
                    if ev.kind == "tokens":
                        toks += ev.tokens
                        order.append(tag)
                    else:
                        done.add(tag)
                        return toks
            ta, tb = await asyncio.gather(drain("a", qa), drain("b", qb))
            return first.tokens + ta, tb, order
        finally:
            be.shutdown()
    ta, tb, order = asyncio.run(main())
    assert ta == alone[0] and tb == alone[1]
    # the 90-token prompt needs four chunks of <= 23 rows: request a emitted at least three tokens before b's first
    assert order.index("b") >= 3
