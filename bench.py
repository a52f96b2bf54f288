#!/usr/bin/env python
"""Headline benchmark: greedy decode throughput of the Llama-3-8B-shape decoder.

Config (fixed): 32 layers, hidden 4096, 32 q / 8 kv heads, head_dim 128, SwiGLU 14336, vocab
128256, BF16, random-init N(0, 0.02) weights, 64 sequences with 1024-token synthetic prompts
(seeded uniform ids), paged KV cache with 64-token blocks, tensor parallel over the N GPUs of
one node. A step is one decode step of the whole batch (64 new tokens).

Two numbers are reported:
  * ``value``  -- device-timed: K consecutive decode steps queued without host synchronisation
    (per-step metadata upload + CUDA-graph replay + on-device token feedback), CUDA events,
    max over ranks.
  * ``e2e``    -- the same K steps through the public engine API (`Engine.decode`): every step
    copies its metadata from pinned host memory, replays the graph and reads the sampled ids
    back to the host.
The weights (16 GB per step at N=1) are far larger than the 126 MB L2, so no explicit L2 flush
is needed between steps.

``--impl reference`` would run the reference implementation; it is a Rust crate and cannot be
built in this environment, so that arm prints an ``unavailable`` line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent))


def parse() -> argparse.Namespace:
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=64)
    p.add_argument("--warmup", type=int, default=8)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--model", default="llama3-8b-shape")
    p.add_argument("--batch", type=int, default=64)
    p.add_argument("--prompt", type=int, default=1024)
    p.add_argument("--parallelism", default="tp", choices=["tp", "dp"])
    p.add_argument("--no-graph", action="store_true")
    p.add_argument("--skip-e2e", action="store_true")
    p.add_argument("--device", default="cuda", choices=["cuda", "cpu"], help="cpu is for debugging the harness only")
    return p.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines: list[str] = []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main() -> None:
    args = parse()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference is a Rust crate (cargo/rustc not installed; pip: 'neither setup.py nor "
                          "pyproject.toml found'), it cannot be built or run here"}))
        return

    import torch
    import torch.distributed as dist
    from flyingfish_b200 import ops
    from flyingfish_b200.api import Model
    from flyingfish_b200.config import Settings

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    on_gpu = args.device == "cuda"
    if on_gpu:
        torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank) if on_gpu else torch.device("cpu")
    comm = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
        if args.parallelism == "tp":
            from flyingfish_b200.parallel.comm import TPComm
            from flyingfish_b200.config import named_shape as _ns
            _h = _ns(args.model).hidden
            comm = TPComm.create(dist.group.WORLD, device, slot_bytes=(8192 // world) * _h * 2)

    global_batch = args.batch if (args.parallelism == "tp" or world == 1) else args.batch * world
    local_batch = args.batch
    capacity = ((args.prompt + 2 * (args.warmup + args.steps) + 8 + 63) // 64) * 64
    settings = Settings(device=local_rank, capacity=capacity, max_batch=local_batch, graph=not args.no_graph,
                        tp=world if comm is not None else 1)
    model = Model.load(args.model, settings, device=device, random_init=True, seed=0, comm=comm)
    eng = model.engine
    spec = model.spec

    g = torch.Generator().manual_seed(1 + (rank if comm is None else 0))
    prompts = [torch.randint(0, spec.vocab, (args.prompt,), generator=g).tolist() for _ in range(local_batch)]
    seqs = [eng.add_sequence(p) for p in prompts]

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        if on_gpu:
            torch.cuda.synchronize(device)

    class Ev:
        """CUDA event on the current stream (wall clock when debugging on a CPU)."""
        def __init__(self):
            self.e = torch.cuda.Event(enable_timing=True) if on_gpu else None
            self.t = 0.0
        def record(self):
            if self.e is not None:
                self.e.record()
            else:
                self.t = time.perf_counter()
        def elapsed_time(self, other) -> float:
            return self.e.elapsed_time(other.e) if self.e is not None else (other.t - self.t) * 1e3

    # ---- prefill (reported, not the headline) ------------------------------------------------
    barrier()
    e0, e1 = Ev(), Ev()
    e0.record()
    eng.prefill(seqs)
    e1.record()
    barrier()
    prefill_ms = e0.elapsed_time(e1)

    # ---- e2e: public API, per-step H2D of metadata + D2H of ids --------------------------------
    e2e = None
    launches_per_step = None
    if not args.skip_e2e:
        for _ in range(args.warmup):
            eng.decode(seqs)
        ops.reset_launch_count()
        barrier()
        sampler = ClockSampler(local_rank); sampler.start()
        e0.record()
        for _ in range(args.steps):
            eng.decode(seqs)
        e1.record()
        barrier()
        clocks_e2e = sampler.stop()
        ms = e0.elapsed_time(e1)
        t = torch.tensor([ms], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item()) / args.steps
        from flyingfish_b200.engine.engine import bucket_for as _bf
        fbb = eng._decode_batch(_bf(local_batch))
        e2e = {"value": global_batch / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": fbb.h2d_bytes(), "d2h_bytes_per_step": 4 * fbb.layout.max_batch,
               "clocks": clocks_e2e}

    # ---- device-timed: K steps queued back to back ----------------------------------------------
    from flyingfish_b200.engine.engine import bucket_for
    bucket = bucket_for(local_batch)
    if eng.use_graph:
        gr = eng.capture(bucket)
        fb = gr.batch
    else:
        gr = None
        fb = eng._decode_batch(bucket)
    total_steps = args.warmup + args.steps
    # precompute per-step metadata on the host (positions/slots/ctx are predictable; ids are fed
    # back on the device from the previous step's output)
    L = fb.layout
    staged = torch.empty(total_steps, L.total, dtype=torch.int32, pin_memory=on_gpu)
    for i in range(total_steps):
        eng._fill_decode(fb, seqs, bucket)
        staged[i].copy_(fb.host)
        for s in seqs:
            eng.kv.commit(s.seq_id, 1)
    last = torch.tensor([s.pending for s in seqs] + [0] * (bucket - len(seqs)), dtype=torch.int32, device=device)
    ids_view = fb.dev[L.ids: L.ids + bucket]

    def one_step(i: int, prev: torch.Tensor) -> torch.Tensor:
        fb.dev.copy_(staged[i], non_blocking=True)
        ids_view.copy_(prev)
        if gr is not None:
            gr.graph.replay()
            return gr.out
        return model.engine.model.forward(fb, eng.kv)

    ops.reset_launch_count()
    prev = last
    for i in range(args.warmup):
        prev = one_step(i, prev)
    barrier()
    if gr is None:
        ops.reset_launch_count()
    sampler = ClockSampler(local_rank); sampler.start()
    e0.record()
    for i in range(args.warmup, total_steps):
        prev = one_step(i, prev)
    e1.record()
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    t = torch.tensor([ms], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    if on_gpu:
        ops.check_status(device)

    # launches of this library's kernels per step: counted during an eager step
    eng.use_graph = False
    ops.reset_launch_count()
    fb2 = eng._decode_batch(bucket)
    fb2.host.copy_(staged[total_steps - 1]); fb2.rows = bucket; fb2.batch = bucket; fb2.n_logit_rows = bucket
    fb2.is_decode = True; fb2.nq = 1; fb2.max_ctx = capacity; fb2.use_tree_mask = False
    fb2.upload()
    eng.model.forward(fb2, eng.kv)
    if on_gpu:
        torch.cuda.synchronize(device)
    launches_per_step = ops.launch_count()

    value = global_batch / (ms_per_step / 1e3)
    weight_bytes = spec.decode_weight_bytes() / (world if comm is not None else 1)
    kv_bytes = local_batch * (args.prompt + args.warmup + args.steps / 2) * spec.layers * 2 * \
        (max(1, spec.kv_heads // (world if comm is not None else 1))) * spec.head_dim * 2
    roof = (weight_bytes + kv_bytes) / (ms_per_step / 1e3) / 1e9
    peaks = {}
    pk = Path(__file__).resolve().parent / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
    hbm = peaks.get("hbm_gbs", 6650.0)
    if rank == 0:
        out = {
            "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if args.parallelism == "tp" else "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded uniform token ids, random-init N(0,0.02) weights)",
            "config": {"model": args.model, "global_batch": global_batch, "seq_len": args.prompt,
                       "new_tokens_timed": args.steps, "kv_block": 64,
                       "parallelism": f"{args.parallelism}{world}", "graph": eng.graphs != {},
                       "l2": "inputs larger than L2 (weights + KV read per step >> 126 MB)"},
            "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
            "launches_per_step": launches_per_step,
            "prefill_tokens_per_s": global_batch * args.prompt / (prefill_ms / 1e3),
            "hbm_gbs_achieved": roof, "hbm_frac_of_measured": roof / hbm,
            "impl": "ours",
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
