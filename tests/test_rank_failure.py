"""A rank that leaves between steps: the survivors' next collective ends with an error (the failure is made on the
host: the rank simply exits; nothing on a device faults or hangs), the engine poisons itself, the serving backend fails
the request in flight and reports ``unavailable`` from then on. Two gloo ranks on CPU with a short process-group
time-out run the tensor-parallel tiny decoder."""
import asyncio
import multiprocessing as mp
import os
from datetime import timedelta

import pytest


def _rank(rank: int, port: int, q) -> None:
    import torch
    import torch.distributed as dist
    from flyingfish_b200.api import Model
    from flyingfish_b200.config import Settings
    from flyingfish_b200.engine.engine import EnginePoisoned
    from flyingfish_b200.parallel.comm import TPComm
    from flyingfish_b200.serve.backend import Backend, Unavailable
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE="2")
    dist.init_process_group("gloo", rank=rank, world_size=2, timeout=timedelta(seconds=8))
    comm = TPComm.create(dist.group.WORLD, torch.device("cpu"))
    model = Model.load("tiny-llama", Settings(capacity=128, max_batch=2, graph=False), device="cpu", seed=0, comm=comm)
    eng = model.engine
    seq = eng.add_sequence(list(range(4, 30)))
    toks = eng.prefill([seq])
    for _ in range(3):
        toks = eng.decode([seq])
    eng.free_sequence(seq.seq_id)
    dist.barrier()
    if rank == 1:
        # leaves between steps: nothing of its own is in flight
        q.put((1, "left"))
        q.close(); q.join_thread()
        os._exit(0)

    async def serve_after_peer_left():
        backend = Backend(eng, eos_ids=())
        backend.start()
        try:
            req, events = backend.add_request(list(range(5, 20)), 4, ignore_eos=True)
            ev = await asyncio.wait_for(events.get(), timeout=60)
            first = ev.kind
            for _ in range(100):
                if backend.state == "unavailable":
                    break
                await asyncio.sleep(0.05)
            try:
                backend.add_request([1, 2, 3], 2)
                second = "accepted"
            except Unavailable:
                second = "unavailable"
            return first, backend.state, second
        finally:
            backend.shutdown()
    import time
    time.sleep(1.0)
    res = asyncio.run(serve_after_peer_left())
    try:
        eng.add_sequence([1, 2, 3])
        poisoned = False
    except EnginePoisoned:
        poisoned = True
    q.put((0, res, poisoned))
    q.close(); q.join_thread()
    os._exit(0)


def test_peer_leaving_between_steps_poisons_and_marks_unavailable():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, 29641, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        item = q.get(timeout=240)
        got[item[0]] = item[1:]
    for p in procs:
        p.join(timeout=60)
    assert got[1] == ("left",)
    (first_event, state, second), poisoned = got[0]
    assert first_event == "failed"            # the request in flight ends with an error (HTTP 500 at the server)
    assert state == "unavailable" and second == "unavailable"
    assert poisoned
