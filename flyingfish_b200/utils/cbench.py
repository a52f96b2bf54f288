"""Benchmark of the fused compute+collective kernels against their roofline and against the unfused
path (this library's GEMM followed by an NCCL collective).

Launch one rank per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m flyingfish_b200.utils.cbench --iters 30

Every number is device time (CUDA events on the launching stream, after warm-up, a barrier and a
synchronise on both sides) and the maximum over ranks. Between timed launches a buffer larger than
L2 is rewritten. Roofline of a kernel = the slowest of its FLOPs at the measured GEMM peak, its HBM
bytes at the measured copy bandwidth and the bytes a rank must move over NVLink at the measured
770 GB/s per direction; ``frac`` = roofline time / achieved time.

Kernels: ``gemm_ar`` (row-parallel projection + one-shot all-reduce, decode sizes), ``ag_gemm``
(all-gather -> GEMM, prefill), ``gemm_rs`` (GEMM -> reduce-scatter, prefill).
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0          # measured peer copy, per direction per GPU
NVLINK_NOMINAL_GBS = 900.0  # NVLink 5 nominal, per direction per GPU: fractions are reported against both
ROOT = Path(__file__).resolve().parents[2]


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "tflops": 1590.0, "source": "fallback"}


def timed(fn, iters: int, warmup: int, flush: torch.Tensor, device) -> float:
    """Mean device time of ``fn`` in microseconds, max over ranks."""
    for _ in range(warmup):
        fn()
    dist.barrier()
    torch.cuda.synchronize(device)
    total = 0.0
    for _ in range(iters):
        for _ in range(2):
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize(device)
        total += e0.elapsed_time(e1) * 1e3
    t = torch.tensor([total / iters], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.barrier()
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--iters", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--decode-rows", type=int, default=64)
    ap.add_argument("--prefill-rows", type=int, default=8192, help="total rows of the sequence-parallel prefill chunk")
    ap.add_argument("--kernels", default="gemm_ar,ag_gemm,gemm_rs", help="comma-separated subset to run")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    from .. import ops
    from ..parallel.comm import TPComm
    h, f = args.hidden, args.ffn
    rpr = args.prefill_rows // world
    comm = TPComm.create(dist.group.WORLD, device, slot_bytes=rpr * h * 2)
    comm.sp_fused = True          # this tool times the one-kernel forms at every world size
    pk = peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    g = torch.Generator(device="cpu").manual_seed(3)
    rnd = lambda *s: (torch.randn(*s, generator=g) * 0.05).to(torch.bfloat16).to(device)
    rows = []

    def report(name, shape, t_us, flops, hbm_bytes, nvl_bytes, t_unfused):
        t_c, t_h, t_n = flops / (pk["tflops"] * 1e6), hbm_bytes / (pk["hbm_gbs"] * 1e3), nvl_bytes / (NVLINK_GBS * 1e3)
        roof = max(t_c, t_h, t_n)
        roof900 = max(t_c, t_h, nvl_bytes / (NVLINK_NOMINAL_GBS * 1e3))
        rows.append({"kernel": name, "shape": shape, "world": world, "us": round(t_us, 2), "unfused_us": round(t_unfused, 2),
                     "roof_us": round(roof, 2), "bound": ["tensor", "hbm", "nvlink"][[t_c, t_h, t_n].index(roof)],
                     "frac_of_roofline": round(roof / t_us, 3), "frac_of_roofline_900": round(roof900 / t_us, 3),
                     "speedup_vs_unfused": round(t_unfused / t_us, 2),
                     "peaks": pk["source"]})

    # ---- decode: row-parallel projection + all-reduce ---------------------------------------
    m = args.decode_rows
    want = set(args.kernels.split(","))
    for (n, k_total, label) in [(h, h, "o_proj"), (h, f, "down_proj")] if "gemm_ar" in want else []:
        k = k_total // world
        x, w = rnd(m, k), rnd(n, k)
        t = timed(lambda: comm.row_linear(x, w), args.iters, args.warmup, flush, device)

        def unfused():
            y = ops.linear(x, w)
            dist.all_reduce(y)
            return y
        tu = timed(unfused, args.iters, args.warmup, flush, device)
        report("gemm_ar", f"{label} M{m} N{n} K{k}", t, 2.0 * m * n * k, (n * k + m * k + m * n) * 2.0,
               (world - 1) * m * n * 2.0, tu)

    # ---- prefill: all-gather -> GEMM (column-parallel) and GEMM -> reduce-scatter (row-parallel)
    mt = args.prefill_rows
    if comm.sp_ok(mt, h, h):
        for (n_total, label) in [(3 * h // 2, "qkv"), (2 * f, "gate_up")] if "ag_gemm" in want else []:
            n = n_total // world
            xs, w = rnd(rpr, h), rnd(n, h)
            t = timed(lambda: comm.ag_linear(xs, w), max(args.iters // 3, 5), 3, flush, device)

            def unfused_ag():
                return ops.linear(comm.all_gather_rows(xs), w)
            tu = timed(unfused_ag, max(args.iters // 3, 5), 3, flush, device)
            report("ag_gemm", f"{label} M{mt} N{n} K{h}", t, 2.0 * mt * n * h, (n * h + mt * h + mt * n) * 2.0,
                   (world - 1) * rpr * h * 2.0, tu)
        for (k_total, label) in [(h, "o_proj"), (f, "down_proj")] if "gemm_rs" in want else []:
            k = k_total // world
            x, w = rnd(mt, k), rnd(h, k)
            t = timed(lambda: comm.rs_linear(x, w), max(args.iters // 3, 5), 3, flush, device)

            def unfused_rs():
                y = ops.linear(x, w)
                out = torch.empty(rpr, h, dtype=y.dtype, device=device)
                dist.reduce_scatter_tensor(out, y)
                return out
            tu = timed(unfused_rs, max(args.iters // 3, 5), 3, flush, device)
            report("gemm_rs", f"{label} M{mt} N{h} K{k}", t, 2.0 * mt * h * k, (h * k + mt * k + rpr * h) * 2.0,
                   (world - 1) * rpr * h * 2.0, tu)
    ops.check_status(device)
    if rank == 0:
        for r in rows:
            print(json.dumps(r))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
