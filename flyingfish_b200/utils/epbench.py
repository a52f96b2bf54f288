"""Benchmark of the expert-parallel MoE layer (dispatch -> grouped expert GEMMs -> combine over peer memory)
against its roofline and against the library path (NCCL all-to-all of the same payload around the same GEMMs).

Launch one rank per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m flyingfish_b200.utils.epbench --rows 4096 --iters 20

Every number is device time (CUDA events on the launching stream after warm-up, a barrier and a synchronise on
both sides), the mean over ``iters`` launches and the maximum over ranks. A buffer larger than L2 is rewritten
between timed launches. Routing is uniform random without replacement (seeded), so a fraction
``(world - 1) / world`` of the assignments crosses NVLink. Roofline of a phase = the slowest of its FLOPs at
the measured GEMM peak, its HBM bytes at the measured copy bandwidth and the bytes a rank must move over NVLink
in one direction at the measured 770 GB/s; ``frac`` = roofline time / achieved time.

Shapes: ``qwen3moe`` (hidden 4096, 128 experts, top-8, expert FFN 1536) and ``dsv3`` (hidden 7168, 256 experts,
top-8, expert FFN 2048); ``--experts`` lowers the expert count when the weights of all local experts should
stay small.
"""
from __future__ import annotations

import argparse
import json
import os
from types import SimpleNamespace

import torch
import torch.distributed as dist

from .cbench import NVLINK_GBS, peaks

SHAPES = {"qwen3moe": (4096, 128, 8, 1536), "dsv3": (7168, 256, 8, 2048)}


def timed(fn, pre, iters: int, warmup: int, flush: torch.Tensor, device) -> float:
    """Mean device time of ``fn`` in microseconds (max over ranks); ``pre`` runs untimed before every launch."""
    total = 0.0
    for i in range(warmup + iters):
        pre()
        flush.zero_()
        flush.zero_()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize(device)
        if i >= warmup:
            total += e0.elapsed_time(e1) * 1e3
    t = torch.tensor([total / iters], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--shape", choices=sorted(SHAPES), default="qwen3moe")
    ap.add_argument("--rows", type=int, default=4096, help="token rows per rank")
    ap.add_argument("--experts", type=int, default=0, help="override the expert count (0 = the shape's)")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    from .. import ops
    from ..parallel.ep import EPComm
    hidden, E, k, f = SHAPES[args.shape]
    E = args.experts or E
    rows, El = args.rows, E // world
    ep = EPComm(dist.group.WORLD, device, E, hidden, max_rows=rows, top_k=k, inter=f)
    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    g = torch.Generator(device="cpu").manual_seed(11 + rank)
    x = (torch.randn(rows, hidden, generator=g) * 0.5).to(torch.bfloat16).to(device)
    ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(rows)]).to(torch.int32).to(device)
    wts = torch.softmax(torch.randn(rows, k, generator=g), -1).to(device)
    gw = torch.Generator(device=device).manual_seed(5)
    lw = SimpleNamespace(
        experts_gu=torch.randn(El, 2 * f, hidden, generator=gw, device=device, dtype=torch.bfloat16) * 0.02,
        experts_down=torch.randn(El, hidden, f, generator=gw, device=device, dtype=torch.bfloat16) * 0.02)
    state = {}

    def do_dispatch():
        state["pos"] = ep.dispatch(x, ids)

    def do_experts():
        ep.experts(lw)

    def do_combine():
        state["out"] = ep.combine(state["pos"], ids, wts, rows)

    def whole():
        state["out"] = ep.dispatch_ffn_combine(x, wts, ids, lw, 0)

    nothing = lambda: None
    # the three phases of one layer call, timed one by one (every rank runs them in the same order)
    tot = {"dispatch": 0.0, "experts": 0.0, "combine": 0.0}
    for i in range(args.warmup + args.iters):
        for name, fn in (("dispatch", do_dispatch), ("experts", do_experts), ("combine", do_combine)):
            flush.zero_()
            flush.zero_()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize(device)
            if i >= args.warmup:
                tot[name] += e0.elapsed_time(e1) * 1e3 / args.iters
    t = torch.tensor([tot["dispatch"], tot["experts"], tot["combine"]], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    t_disp, t_exp, t_comb = (float(v) for v in t.tolist())
    t_whole = timed(whole, nothing, args.iters, args.warmup, flush, device)

    # library path: equal-split all-to-all of the dispatched rows and of the expert outputs
    n_cross = rows * k
    send = torch.empty(n_cross, hidden, dtype=torch.bfloat16, device=device)
    recv = torch.empty_like(send)
    t_a2a = timed(lambda: dist.all_to_all_single(recv, send), nothing, args.iters, args.warmup, flush, device)

    cross = rows * k * (world - 1) / world * hidden * 2.0          # bytes over NVLink, one direction, per phase
    recv_rows = rows * k                                             # uniform routing: what a rank's experts receive
    flops = 2.0 * recv_rows * hidden * 2 * f + 2.0 * recv_rows * f * hidden
    w_bytes = El * 3.0 * f * hidden * 2
    act = recv_rows * hidden * 2.0
    us = lambda b, bw: b / (bw * 1e3)
    roof_disp = max(us(cross, NVLINK_GBS), us(rows * hidden * 2.0 + act / world, pk["hbm_gbs"]))
    roof_comb = max(us(cross, NVLINK_GBS), us(act / world + rows * hidden * 2.0, pk["hbm_gbs"]))
    roof_exp = max(flops / (pk["tflops"] * 1e6), us(w_bytes + 2 * act + recv_rows * f * 4.0, pk["hbm_gbs"]))
    roof_whole = roof_disp + roof_exp + roof_comb
    # the same rooflines with NVLink at its nominal 900 GB/s per direction instead of the measured 770
    r9_disp = max(us(cross, 900.0), us(rows * hidden * 2.0 + act / world, pk["hbm_gbs"]))
    r9_comb = max(us(cross, 900.0), us(act / world + rows * hidden * 2.0, pk["hbm_gbs"]))
    roof900 = {"ep_dispatch": r9_disp, "ep_experts": roof_exp, "ep_combine": r9_comb, "ep_layer": r9_disp + roof_exp + r9_comb}
    ops.check_status(device)
    if rank == 0:
        base = {"shape": f"{args.shape} rows{rows}/rank E{E} top{k} hidden{hidden} ffn{f}", "world": world,
                "peaks": pk["source"]}
        for name, tt, roof, unf in (("ep_dispatch", t_disp, roof_disp, t_a2a), ("ep_experts", t_exp, roof_exp, None),
                                    ("ep_combine", t_comb, roof_comb, t_a2a),
                                    ("ep_layer", t_whole, roof_whole, t_exp + 2 * t_a2a)):
            row = {"kernel": name, **base, "us": round(tt, 1), "roof_us": round(roof, 1),
                   "frac_of_roofline": round(roof / tt, 3), "frac_of_roofline_900": round(roof900[name] / tt, 3)}
            if unf is not None:
                row["nccl_all_to_all_us" if name != "ep_layer" else "library_path_us"] = round(unf, 1)
                row["speedup_vs_library"] = round(unf / tt, 2)
            print(json.dumps(row))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
