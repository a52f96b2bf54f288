#!/usr/bin/env python
"""Headline benchmark: greedy decode throughput of a dense decoder, tensor parallel over N GPUs.

Default config (``--config 2``): Llama-3-8B shape -- 32 layers, hidden 4096, 32 q / 8 kv heads,
head_dim 128, SwiGLU 14336, vocab 128256, BF16, random-init N(0, 0.02) weights, 64 sequences with
1024-token synthetic prompts (seeded uniform ids), paged KV cache with 64-token blocks, tensor
parallel over the N GPUs of one node. ``--config 3`` selects the Llama-3-70B shape (batch 32,
prompt 4096). A step is one decode step of the whole batch.

Three arms (``--impl``):
  * ``ours``      -- this framework's engine and kernels. Reports
      ``value``  device-timed: K decode steps queued without host synchronisation (per-step
                 metadata upload + CUDA-graph replay + on-device token feedback), CUDA events,
                 max over ranks;
      ``e2e``    the same K steps through the public engine API (``Engine.decode``): every step
                 copies its metadata from pinned host memory, replays the graph and reads the
                 sampled ids back to the host;
      ``ttft_p50_ms``  median time to first token of ``batch`` requests submitted together to
                 the continuous-batching scheduler;
      ``other_batches``  device-timed decode at the other batch sizes of the config;
      ``baseline`` / ``vs_baseline``  unless ``--skip-baseline``: the library-call arm below
                 measured in the same process on the same GPUs, and e2e(ours) / e2e(baseline).
  * ``baseline``  -- the same model from vendor libraries only (cuBLAS matmul, flash-attn or SDPA
                 attention, NCCL all-reduce, one CUDA graph per step): ``baseline/torch_decoder.py``.
  * ``reference`` -- the reference implementation is a Rust crate and cannot be built in this
                 environment; the arm prints an ``unavailable`` line.

The weights read per step (16 GB at N=1) are far larger than the 126 MB L2, so no explicit L2
flush is needed between steps. SM clocks and throttle reasons are sampled with nvidia-smi every
10 ms from before the warm-up on; the samples that fall inside each timed region are summarised.
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

CONFIGS = {
    2: {"model": "llama3-8b-shape", "batch": 64, "prompt": 1024, "batches": (1, 8, 64), "parallelism": "tp"},
    3: {"model": "llama3-70b-shape", "batch": 32, "prompt": 4096, "batches": (1, 32, 128), "parallelism": "tp"},
    # DeepSeek-V3 shape: FP8 E4M3 weights with 128x128 block scales, MLA, expert parallel over the N GPUs (attention
    # data parallel: every rank serves batch / N sequences), one MTP module
    4: {"model": "deepseek-v3-shape", "batch": 64, "prompt": 1024, "batches": (1, 64, 256), "parallelism": "ep"},
    # Qwen3-MoE-235B shape: NVFP4 experts, expert parallel, half of every rank's experts resident in GPU slots and
    # the rest in the pinned host tier
    5: {"model": "qwen3-moe-235b-shape", "batch": 128, "prompt": 1024, "batches": (128,), "parallelism": "ep",
        "resident": 0.5},
}


def parse() -> argparse.Namespace:
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=64)
    p.add_argument("--warmup", type=int, default=8)
    p.add_argument("--impl", default="ours", choices=["ours", "baseline", "reference"])
    p.add_argument("--config", type=int, default=2, choices=sorted(CONFIGS))
    p.add_argument("--model", default=None)
    p.add_argument("--batch", type=int, default=None)
    p.add_argument("--prompt", type=int, default=None)
    p.add_argument("--layers", type=int, default=None, help="run a reduced-depth variant (reported in config)")
    p.add_argument("--parallelism", default=None, choices=["tp", "dp", "ep"])
    p.add_argument("--resident", type=float, default=None, help="fraction of the experts kept in GPU slots (config 5)")
    p.add_argument("--mtp", type=int, default=0, help="also time MTP speculation of this depth (config 4)")
    p.add_argument("--no-graph", action="store_true")
    p.add_argument("--skip-e2e", action="store_true")
    p.add_argument("--skip-baseline", action="store_true")
    p.add_argument("--skip-extras", action="store_true", help="no TTFT run and no other batch sizes")
    p.add_argument("--device", default="cuda", choices=["cuda", "cpu"], help="cpu is for debugging the harness only")
    a = p.parse_args()
    c = CONFIGS[a.config]
    a.model = a.model or c["model"]
    a.batch = a.batch or c["batch"]
    a.prompt = a.prompt or c["prompt"]
    a.batches = c["batches"]
    a.parallelism = a.parallelism or c["parallelism"]
    if a.resident is None:
        a.resident = c.get("resident")
    if a.parallelism == "ep":
        a.skip_baseline = True          # the library-call arm models the dense decoder only
    return a


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi for the life of the process; ``window`` summarises the
    samples whose arrival time falls inside a timed region (plus the nearest sample on each side, since a region can
    be shorter than a few polling intervals)."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, gpu_index: int, period_ms: int = 10):
        self.gpu, self.period_ms = gpu_index, period_ms
        self.proc = None
        self.samples: list[tuple[float, float, float, tuple[str, ...]]] = []

    def start(self) -> None:
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms),
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self) -> None:
        assert self.proc is not None and self.proc.stdout is not None
        for line in self.proc.stdout:
            now = time.perf_counter()
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm, mx = float(f[1]), float(f[2])
            except ValueError:
                continue
            reasons = tuple(n for n, v in zip(self.NAMES, f[5:9]) if v.lower().startswith("active"))
            self.samples.append((now, sm, mx, reasons))

    def wait_first(self, timeout: float = 5.0) -> None:
        t0 = time.perf_counter()
        while self.proc is not None and not self.samples and time.perf_counter() - t0 < timeout:
            time.sleep(0.02)

    def window(self, t0: float, t1: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        snap = list(self.samples)
        inside = [s for s in snap if t0 <= s[0] <= t1]
        # the polling process delivers a line a little after it sampled: also take the first line after the region
        after = [s for s in snap if s[0] > t1][:1]
        sel = inside + after
        if not sel:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no sample inside the region"], "samples": 0,
                    "region_ms": (t1 - t0) * 1e3}
        reasons = sorted({r for s in sel for r in s[3]})
        return {"sm_mhz": statistics.median(s[1] for s in sel), "sm_max_mhz": max(s[2] for s in sel),
                "reasons": reasons, "samples": len(sel), "region_ms": (t1 - t0) * 1e3}

    def stop(self) -> None:
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()


class Ctx:
    """Process-wide handles shared by the arms."""
    def __init__(self, args):
        import torch
        import torch.distributed as dist
        self.torch, self.dist, self.args = torch, dist, args
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus and self.world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
        self.on_gpu = args.device == "cuda"
        if self.on_gpu:
            torch.cuda.set_device(self.local_rank)
        self.device = torch.device("cuda", self.local_rank) if self.on_gpu else torch.device("cpu")
        if self.world > 1:
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            # NCCL's own log lines (version banner) go to stderr: stdout carries exactly one JSON line
            os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
            dist.init_process_group("nccl" if self.on_gpu else "gloo", device_id=self.device if self.on_gpu else None)
        self.sampler = ClockSampler(self.local_rank)
        if self.on_gpu:
            self.sampler.start()

    def barrier(self) -> None:
        if self.world > 1:
            self.dist.barrier()
        if self.on_gpu:
            self.torch.cuda.synchronize(self.device)

    def max_over_ranks(self, ms: float) -> float:
        if self.world == 1:
            return ms
        t = self.torch.tensor([ms], device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def event(self):
        torch = self.torch
        on_gpu = self.on_gpu

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
        return Ev()

    def timed(self, fn, steps: int) -> tuple[float, dict]:
        """Barrier + synchronise, ``steps`` calls of ``fn(i)`` between two events, barrier + synchronise; returns
        (ms per step as the max over ranks, clock summary of the region)."""
        e0, e1 = self.event(), self.event()
        self.barrier()
        t0 = time.perf_counter()
        e0.record()
        for i in range(steps):
            fn(i)
        e1.record()
        self.barrier()
        t1 = time.perf_counter()
        return self.max_over_ranks(e0.elapsed_time(e1)) / steps, self.sampler.window(t0, t1)


def spec_for(args):
    from flyingfish_b200.config import named_shape
    spec = named_shape(args.model)
    if args.layers:
        spec.layers = args.layers
    return spec


# ------------------------------------------------------------------------------------------------
# this framework
# ------------------------------------------------------------------------------------------------
def run_ours(cx: Ctx) -> dict:
    args, torch, dist = cx.args, cx.torch, cx.dist
    from flyingfish_b200 import ops
    from flyingfish_b200.api import Model
    from flyingfish_b200.config import Settings
    from flyingfish_b200.engine.engine import bucket_for
    from flyingfish_b200.engine.scheduler import Request, Scheduler

    world, rank, device, on_gpu = cx.world, cx.rank, cx.device, cx.on_gpu
    spec0 = spec_for(args)
    comm, ep = None, None
    if world > 1 and args.parallelism == "tp":
        from flyingfish_b200.parallel.comm import TPComm
        comm = TPComm.create(dist.group.WORLD, device, slot_bytes=(8192 // world) * spec0.hidden * 2)
    tp = world if comm is not None else 1
    if args.parallelism == "ep":
        # experts sharded over the ranks, attention data parallel: the batch is split over the ranks
        global_batch = args.batch
        local_batch = max(1, args.batch // world)
        if world > 1:
            from flyingfish_b200.parallel.ep import EPComm
            ep = EPComm(dist.group.WORLD, device, spec0.moe.num_experts, spec0.hidden,
                        max_rows=max(local_batch, 8192 // 8), top_k=spec0.moe.top_k)
    else:
        global_batch = args.batch if (args.parallelism == "tp" or world == 1) else args.batch * world
        local_batch = args.batch
    max_batch = max([local_batch] + ([] if args.skip_extras else list(args.batches)))
    capacity = ((args.prompt + 2 * (args.warmup + args.steps) + 8 + 63) // 64) * 64
    settings = Settings(device=cx.local_rank, capacity=capacity, max_batch=max_batch, graph=not args.no_graph, tp=tp)
    model = Model.load(args.model if not args.layers else spec0, settings, device=device, random_init=True, seed=0,
                       comm=comm, ep=ep)
    eng, spec = model.engine, model.spec
    provider = None
    if args.resident is not None and spec.moe is not None:
        from flyingfish_b200.experts.provider import build_provider_from_weights
        provider = build_provider_from_weights(eng.model, resident_fraction=args.resident, threads=8, settings=settings)
        if ep is not None:
            ep.provider = provider
        provider.collect_freq = True
    g = torch.Generator().manual_seed(1 + (rank if comm is None else 0))

    def new_prompts(n: int) -> list[list[int]]:
        return [torch.randint(0, spec.vocab, (args.prompt,), generator=g).tolist() for _ in range(n)]

    # ---- p50 time to first token: `batch` requests arrive together at the continuous-batching scheduler ----------
    ttft = None
    if not args.skip_extras:
        sch = Scheduler(eng)
        reqs = [Request(prompt=p, max_tokens=1, ignore_eos=True) for p in new_prompts(local_batch)]
        cx.barrier()
        for r in reqs:
            r.arrival = time.perf_counter()
            sch.submit(r)
        sch.run_until_idle()
        cx.barrier()
        t = sorted(r.ttft_ms for r in reqs if r.ttft_ms is not None)
        ttft = cx.max_over_ranks(t[len(t) // 2]) if t else None
        eng.reset()

    seqs = [eng.add_sequence(p) for p in new_prompts(local_batch)]

    # ---- prefill (reported, not the headline) ---------------------------------------------------------------------
    prefill_ms, _ = cx.timed(lambda i: eng.prefill(seqs), 1)
    if provider is not None:
        # slots are filled by the prefill's routing frequency, as at a request boundary
        provider.collect_freq = False
        provider.begin_request()
        for k in ("hits", "host_misses", "disk_misses"):
            provider.res.stats[k] = 0

    # ---- e2e: public API, per-step H2D of metadata + D2H of ids -----------------------------------------------------
    e2e = None
    if not args.skip_e2e:
        for _ in range(args.warmup):
            eng.decode(seqs)
        e2e_ms, clocks_e2e = cx.timed(lambda i: eng.decode(seqs), args.steps)
        fbb = eng._decode_batch(bucket_for(local_batch))
        e2e = {"value": global_batch / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": fbb.h2d_bytes(), "d2h_bytes_per_step": 4 * fbb.layout.max_batch,
               "clocks": clocks_e2e}

    # ---- device-timed: K steps queued back to back ----------------------------------------------------------------
    def device_timed(seqs_, n_local: int, warmup: int, steps: int) -> tuple[float, dict]:
        bucket = bucket_for(n_local)
        if eng.use_graph:
            gr = eng.capture(bucket)
            fb = gr.batch
        else:
            gr = None
            fb = eng._decode_batch(bucket)
        total_steps = warmup + steps
        # per-step metadata precomputed on the host (positions / slots / context lengths are predictable; the ids
        # are fed back on the device from the previous step's output)
        L = fb.layout
        staged = torch.empty(total_steps, L.total, dtype=torch.int32, pin_memory=on_gpu)
        for i in range(total_steps):
            eng._fill_decode(fb, seqs_, bucket)
            staged[i].copy_(fb.host)
            for s in seqs_:
                eng.kv.commit(s.seq_id, 1)
        last = torch.tensor([s.pending for s in seqs_] + [0] * (bucket - len(seqs_)), dtype=torch.int32, device=device)
        ids_view = fb.dev[L.ids: L.ids + bucket]
        state = {"prev": last}

        def one_step(i: int) -> None:
            fb.dev.copy_(staged[i], non_blocking=True)
            ids_view.copy_(state["prev"])
            if gr is not None:
                gr.graph.replay()
                state["prev"] = gr.out
            else:
                state["prev"] = eng.model.forward(fb, eng.kv)

        for i in range(warmup):
            one_step(i)
        ms, clk = cx.timed(lambda i: one_step(warmup + i), steps)
        if on_gpu:
            ops.check_status(device)
        return ms, clk, staged[total_steps - 1], bucket

    if provider is not None:
        # the host tier is serviced inside every step (a device-to-host summary per MoE layer), so there is no
        # host-free form of the step: the device-timed value is the engine step itself
        for _ in range(args.warmup):
            eng.decode(seqs)
        ms_per_step, clocks = cx.timed(lambda i: eng.decode(seqs), args.steps)
        bucket, last_meta = bucket_for(local_batch), None
    else:
        ms_per_step, clocks, last_meta, bucket = device_timed(seqs, local_batch, args.warmup, args.steps)

    # launches of this library's kernels per step: counted during one eager step
    was_graph = eng.use_graph
    eng.use_graph = False
    ops.reset_launch_count()
    if last_meta is None:
        eng.decode(seqs)
    else:
        fb2 = eng._decode_batch(bucket)
        fb2.host.copy_(last_meta); fb2.rows = bucket; fb2.batch = bucket; fb2.n_logit_rows = bucket
        fb2.is_decode = True; fb2.nq = 1; fb2.max_ctx = capacity; fb2.use_tree_mask = False
        fb2.upload()
        eng.model.forward(fb2, eng.kv)
    if on_gpu:
        torch.cuda.synchronize(device)
    launches_per_step = ops.launch_count()
    eng.use_graph = was_graph

    # ---- MTP speculation (config 4): tokens per second of one sequence with the MTP module drafting ---------------
    mtp = None
    if args.mtp > 0:
        from flyingfish_b200.spec.mtp import MtpSpeculator
        eng.reset()
        sp = MtpSpeculator(model, depth=args.mtp, seed=11)
        n_new = max(8, args.steps)
        sp.generate(new_prompts(1)[0], 4)                 # warm-up: captures the verification graph of this row count
        eng.reset()
        sp = MtpSpeculator(model, depth=args.mtp, seed=11)
        cx.barrier()
        t0 = time.perf_counter()
        out = sp.generate(new_prompts(1)[0], n_new)
        cx.barrier()
        dt = time.perf_counter() - t0
        mtp = {"depth": args.mtp, "tokens": len(out.ids), "tokens_per_s": len(out.ids) / max(dt - out.prefill_ms / 1e3, 1e-9),
               "ms_per_round": (dt * 1e3 - out.prefill_ms) / max(sp.stats.rounds, 1),
               "verify_graph_replays": eng.stats.get("verify_graph_replays", 0),
               "rounds": sp.stats.rounds, "acceptance_rate": sp.stats.acceptance_rate,
               "note": "random-init MTP module: acceptance is near zero, the figure is the cost of a round"}

    # ---- the other batch sizes of the config (device-timed only) ----------------------------------------------------
    others = {}
    if not args.skip_extras and provider is None and args.mtp == 0:
        for b in args.batches:
            if b == local_batch or b > max_batch:
                continue
            eng.reset()
            sq = [eng.add_sequence(p) for p in new_prompts(b)]
            eng.prefill(sq)
            ms_b, clk_b, _, _ = device_timed(sq, b, max(3, args.warmup // 2), max(8, args.steps // 2))
            others[str(b)] = {"decode_tokens_per_s": b / (ms_b / 1e3), "ms_per_step": ms_b, "clocks": clk_b}

    value = global_batch / (ms_per_step / 1e3)
    weight_bytes = spec.decode_weight_bytes() / tp
    kv_bytes = local_batch * (args.prompt + args.warmup + args.steps / 2) * spec.layers * 2 * \
        (max(1, spec.kv_heads // tp)) * spec.head_dim * 2
    roof = (weight_bytes + kv_bytes) / (ms_per_step / 1e3) / 1e9
    peaks = {}
    pk = Path(__file__).resolve().parent / "MEASURED_PEAKS.json"
    if pk.exists():
        peaks = json.loads(pk.read_text())
    hbm = peaks.get("hbm_gbs", 6650.0)
    out = {
        "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if args.parallelism in ("tp", "ep") else "weak", "vs_baseline": None,
        "dtype": "bf16" if spec.linear_format == "bf16" else f"{spec.linear_format} weights (W8A8), bf16 activations",
        "data": "synthetic (seeded uniform token ids, random-init N(0,0.02) weights)",
        "config": {"model": args.model, "layers": spec.layers, "global_batch": global_batch, "seq_len": args.prompt,
                   "new_tokens_timed": args.steps, "kv_block": 64,
                   "parallelism": f"{args.parallelism}{world}", "graph": eng.graphs != {},
                   "l2": "inputs larger than L2 (weights + KV read per step >> 126 MB)"},
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * args.steps,
        "launches_per_step": launches_per_step,
        "prefill_tokens_per_s": global_batch * args.prompt / (prefill_ms / 1e3),
        "ttft_p50_ms": ttft, "other_batches": others,
        "hbm_gbs_achieved": roof, "hbm_frac_of_measured": roof / hbm,
        "impl": "ours",
    }
    if spec.moe is not None:
        out["config"].update(experts=spec.moe.num_experts, top_k=spec.moe.top_k, expert_format=spec.moe.expert_format,
                             linear_format=spec.linear_format)
        out.pop("hbm_gbs_achieved"); out.pop("hbm_frac_of_measured")        # the byte model above is the dense decoder's
    if provider is not None:
        st = provider.res.stats
        out["experts"] = {"resident_fraction": args.resident, "slots": "nvfp4" if provider.fp4 else "bf16",
                          "hit_rate": provider.res.hit_rate(), "hits": st["hits"], "host_misses": st["host_misses"],
                          "admitted": st["admitted"], "evicted": st["evicted"], "cpu_rows": provider.stats["cpu_rows"],
                          "gpu_rows": provider.stats["gpu_rows"], "h2d_expert_bytes": provider.stats["h2d_expert_bytes"],
                          "d2h_summary_bytes": provider.stats["d2h_summary_bytes"]}
    if mtp is not None:
        out["mtp"] = mtp
    # release the engine before the comparison arm allocates its own weights
    del model, eng, seqs
    return out


# ------------------------------------------------------------------------------------------------
# library-call baseline
# ------------------------------------------------------------------------------------------------
def run_baseline(cx: Ctx) -> dict:
    args, torch = cx.args, cx.torch
    from baseline.torch_decoder import TorchDecoder
    spec = spec_for(args)
    world, device = cx.world, cx.device
    tp = world if args.parallelism == "tp" else 1
    global_batch = args.batch if (args.parallelism == "tp" or world == 1) else args.batch * world
    capacity = ((args.prompt + 2 * (args.warmup + args.steps) + 8 + 63) // 64) * 64
    net = TorchDecoder(spec, device, args.batch, capacity, rank=cx.rank if tp > 1 else 0, world=tp, seed=0)
    g = torch.Generator().manual_seed(1)
    prompts = torch.randint(0, spec.vocab, (args.batch, args.prompt), generator=g)
    pin = prompts.pin_memory() if cx.on_gpu else prompts

    first = {}

    def do_prefill(i):
        # chunks of sequences keep the activation memory of the library prefill bounded
        outs = []
        step = max(1, 8192 // args.prompt)
        for b0 in range(0, args.batch, step):
            sub = pin[b0: b0 + step].to(device, non_blocking=True)
            saved_k, saved_v = net.k, net.v
            net.k = [k[b0: b0 + step] for k in saved_k]
            net.v = [v[b0: b0 + step] for v in saved_v]
            outs.append(net.prefill(sub))
            net.k, net.v = saved_k, saved_v
        first["ids"] = torch.cat(outs)
    prefill_ms, _ = cx.timed(do_prefill, 1)
    net.lens.fill_(args.prompt)
    net.ids.copy_(first["ids"])
    graph = not args.no_graph
    if graph:
        try:
            net.capture()
        except Exception as e:  # a library that cannot be captured runs eagerly; the arm says so
            graph = False
            net.graph = None
            first["capture_error"] = f"{type(e).__name__}: {e}"[:200]

    # device-timed: ids fed back on the device
    def dev_step(i):
        net.ids.copy_(net.step())
    for i in range(args.warmup):
        dev_step(i)
    ms_per_step, clocks = cx.timed(dev_step, args.steps)

    # end to end: ids come from pinned host memory every step and the sampled ids are read back
    host_ids = torch.zeros(args.batch, dtype=torch.long, pin_memory=cx.on_gpu)
    host_ids.copy_(net.ids.cpu())

    def e2e_step(i):
        net.ids.copy_(host_ids, non_blocking=True)
        out = net.step()
        host_ids.copy_(out.cpu())
    for i in range(min(3, args.warmup)):
        e2e_step(i)
    e2e_ms, clocks_e2e = cx.timed(e2e_step, args.steps)
    return {
        "metric": "decode_tokens_per_s", "value": global_batch / (ms_per_step / 1e3), "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": "strong" if args.parallelism == "tp" else "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (seeded uniform token ids, random-init N(0,0.02) weights)",
        "config": {"model": args.model, "layers": spec.layers, "global_batch": global_batch, "seq_len": args.prompt,
                   "new_tokens_timed": args.steps, "kv": "contiguous", "parallelism": f"{args.parallelism}{world}",
                   "graph": graph, "attention": net.attention_impl, "gemm": "torch.matmul (cuBLAS)",
                   "collectives": "NCCL", "l2": "inputs larger than L2 (weights + KV read per step >> 126 MB)",
                   **({"capture_error": first["capture_error"]} if "capture_error" in first else {})},
        "clocks": clocks,
        "e2e": {"value": global_batch / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": 8 * args.batch, "d2h_bytes_per_step": 8 * args.batch, "clocks": clocks_e2e},
        "gpu_launches": 0, "prefill_tokens_per_s": global_batch * args.prompt / (prefill_ms / 1e3),
        "ttft_p50_ms": prefill_ms, "impl": "baseline",
    }


def main() -> None:
    args = parse()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "reference is a Rust crate (cargo/rustc not installed; pip: 'neither setup.py nor "
                          "pyproject.toml found'), it cannot be built or run here"}))
        return
    cx = Ctx(args)
    cx.sampler.wait_first()
    try:
        if args.impl == "baseline":
            out = run_baseline(cx)
        else:
            out = run_ours(cx)
            if not args.skip_baseline and cx.on_gpu and args.parallelism == "tp":
                import gc
                gc.collect()
                cx.torch.cuda.empty_cache()
                try:
                    base = run_baseline(cx)
                    out["baseline"] = {k: base[k] for k in ("value", "ms_per_step", "e2e", "clocks",
                                                              "prefill_tokens_per_s", "ttft_p50_ms", "config")}
                    if out.get("e2e") and base.get("e2e"):
                        out["vs_baseline"] = out["e2e"]["value"] / base["e2e"]["value"]
                    else:
                        out["vs_baseline"] = out["value"] / base["value"]
                    out["vs_baseline_device_timed"] = out["value"] / base["value"]
                except Exception as e:  # the comparison arm must not take the product's number down with it
                    out["baseline"] = {"error": f"{type(e).__name__}: {e}"[:300]}
        if cx.rank == 0:
            print(json.dumps(out))
    finally:
        cx.sampler.stop()
        if cx.world > 1:
            cx.dist.barrier()
            cx.dist.destroy_process_group()


if __name__ == "__main__":
    main()
