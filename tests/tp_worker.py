"""Worker for the tensor-parallel tests (launched with torch.distributed.run)."""
import argparse
import json
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--out", required=True)
    ap.add_argument("--mode", default="model")
    ap.add_argument("--model", default="qwen3-moe-tiny")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if args.device == "cuda":
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=device)
    else:
        device = torch.device("cpu")
        dist.init_process_group("gloo")
    from flyingfish_b200.parallel.comm import TPComm
    from flyingfish_b200.api import Model
    from flyingfish_b200.config import Settings
    from flyingfish_b200 import ops
    comm = TPComm.create(dist.group.WORLD, device, slot_bytes=8 << 20)
    # routing chosen by world size: one-kernel prefill pair up to four ranks, switch-side all-reduce from eight
    assert comm.sp_fused == (comm.size <= 4) and (not comm.nvls or comm.size >= 4)
    result = {}
    if args.mode == "model":
        m = Model.load("tiny-llama", Settings(capacity=256, max_batch=4, graph=(args.device == "cuda")), device=device,
                       seed=0, comm=comm)
        g = torch.Generator().manual_seed(7)
        prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (40, 9)]
        result["tokens"] = m.generate_batch(prompts, 10)
        result["stats"] = comm.stats
    elif args.mode == "kernels":
        g = torch.Generator().manual_seed(11)
        ok = True
        errs = []
        for (m_, n_, k_) in [(1, 512, 256), (64, 4096, 2048), (17, 1024, 4096), (128, 256, 512)]:
            xs = [(torch.randn(m_, k_, generator=g)).to(torch.bfloat16) for _ in range(world)]
            ws = [(torch.randn(n_, k_, generator=g) * 0.05).to(torch.bfloat16) for _ in range(world)]
            parts = [(xs[r].float() @ ws[r].float().t()).to(torch.bfloat16).float() for r in range(world)]
            expect = sum(parts)
            for rep in range(3):      # repeated launches exercise the epoch / parity protocol
                y = comm.row_linear(xs[rank].to(device), ws[rank].to(device))
                err = (y.float().cpu() - expect).abs().max().item()
                errs.append(err)
                ok = ok and err <= 0.05 + 0.02 * expect.abs().max().item()
            v = torch.randn(m_ * n_, generator=g).to(torch.bfloat16)
            vs = [(v.float() * (r + 1)).to(torch.bfloat16) for r in range(world)]
            yr = comm.all_reduce(vs[rank].to(device).clone())
            exp = sum(t.float() for t in vs)
            err = (yr.float().cpu() - exp).abs().max().item()
            errs.append(err)
            ok = ok and err <= 0.05 + 0.02 * exp.abs().max().item()
        # bitwise identical on every rank
        y = comm.row_linear(xs[rank].to(device), ws[rank].to(device))
        gathered = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(gathered, y)
        same = all(torch.equal(gathered[0], t) for t in gathered)
        if device.type == "cuda":
            torch.cuda.synchronize()
            ops.check_status(device)
        result.update(ok=ok, errs=errs, same=same, stats=comm.stats)
    elif args.mode == "sp":
        # fused all-gather -> GEMM and GEMM -> reduce-scatter against an FP32 reference, repeated
        # launches, then a sequence-parallel prefill of the tiny decoder
        g = torch.Generator().manual_seed(21)
        ok, errs = True, []
        for (m_, n_, k_) in [(256 * world, 512, 256), (128 * world, 768, 1024), (512 * world, 256, 2048)]:
            x = torch.randn(m_, k_, generator=g).to(torch.bfloat16)
            wt = (torch.randn(n_, k_, generator=g) * 0.05).to(torch.bfloat16)
            rpr = m_ // world
            want = (x.float() @ wt.float().t())
            for rep in range(3):
                y = comm.ag_linear(x[rank * rpr: (rank + 1) * rpr].to(device).contiguous(), wt.to(device))
                err = (y.float().cpu() - want).abs().max().item()
                errs.append(err); ok = ok and err <= 0.05 + 0.02 * want.abs().max().item()
            # row-parallel: K split over ranks
            kk = k_ // world
            xs = x[:, rank * kk: (rank + 1) * kk].to(device).contiguous()
            ws_ = wt[:, rank * kk: (rank + 1) * kk].to(device).contiguous()
            parts = [(x[:, r * kk: (r + 1) * kk].float() @ wt[:, r * kk: (r + 1) * kk].float().t()).to(torch.bfloat16).float()
                     for r in range(world)]
            want_rs = sum(parts)[rank * rpr: (rank + 1) * rpr]
            for rep in range(3):
                y = comm.rs_linear(xs, ws_)
                err = (y.float().cpu() - want_rs).abs().max().item()
                errs.append(err); ok = ok and err <= 0.05 + 0.02 * want_rs.abs().max().item()
        m = Model.load("tiny-llama", Settings(capacity=1024, max_batch=4, graph=True), device=device, seed=0, comm=comm)
        gg = torch.Generator().manual_seed(8)
        prompts = [torch.randint(0, 2048, (n,), generator=gg).tolist() for n in (300, 150)]
        toks = m.generate_batch(prompts, 6)
        torch.cuda.synchronize()
        ops.check_status(device)
        result.update(ok=ok, errs=errs, tokens=toks, stats=comm.stats)
    elif args.mode == "ep":
        from flyingfish_b200.parallel.ep import EPComm
        from flyingfish_b200.config import named_shape
        spec = named_shape(args.model)
        ep = EPComm(dist.group.WORLD, device, spec.moe.num_experts, spec.hidden, max_rows=128, top_k=spec.moe.top_k)
        m = Model.load(args.model, Settings(capacity=256, max_batch=4, graph=False), device=device, seed=0, ep=ep)
        g = torch.Generator().manual_seed(100 + rank)       # every rank serves its own sequences
        prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (33, 12)]
        toks = m.generate_batch(prompts, 8)
        gathered = [None] * world
        dist.all_gather_object(gathered, {"prompts": prompts, "tokens": toks})
        if device.type == "cuda":
            torch.cuda.synchronize()
            ops.check_status(device)
        result.update(per_rank=gathered, stats=ep.stats)
    elif args.mode == "ep_skew":
        # receive buffers sized for the balanced share only, every row routed to rank 0's experts: the layer call runs
        # in passes over row slices instead of overflowing
        from types import SimpleNamespace
        from flyingfish_b200.ops import ref
        from flyingfish_b200.parallel.ep import EPComm
        os.environ["FF_EP_ARENA_MAX_GIB"] = "0.00001"
        os.environ["FF_EP_CAPACITY_FACTOR"] = "1"
        E, hidden, inter, top_k, rows = 8, 256, 128, 2, 384
        ep = EPComm(dist.group.WORLD, device, E, hidden, max_rows=rows, top_k=top_k)
        g = torch.Generator().manual_seed(5)
        w_gu = (0.05 * torch.randn(E, 2 * inter, hidden, generator=g)).to(torch.bfloat16)
        w_dn = (0.05 * torch.randn(E, hidden, inter, generator=g)).to(torch.bfloat16)
        gr = torch.Generator().manual_seed(50 + rank)
        n = rows if rank == 0 else rows - 130                      # ranks hold different row counts
        x = torch.randn(n, hidden, generator=gr).to(torch.bfloat16)
        ids = torch.stack([torch.randint(0, 2, (n,), generator=gr), torch.randint(2, 4, (n,), generator=gr)], dim=1).to(torch.int32)
        wts = torch.rand(n, top_k, generator=gr)
        el = E // world
        lw = SimpleNamespace(experts_gu=w_gu[rank * el:(rank + 1) * el].contiguous().to(device),
                             experts_down=w_dn[rank * el:(rank + 1) * el].contiguous().to(device))
        out = ep.dispatch_ffn_combine(x.to(device), wts.to(device), ids.to(device), lw, 0)
        torch.cuda.synchronize()
        ops.check_status(device)
        want = ref.moe_forward(x, wts, ids, w_gu, w_dn, mode=0)
        err = (out.float().cpu() - want.float()).abs().max().item()
        gathered = [None] * world
        dist.all_gather_object(gathered, {"err": err, "scale": want.float().abs().max().item(), "passes": ep.passes,
                                          "worst_case": ep.capacity_is_worst_case, "stats": dict(ep.stats)})
        result.update(per_rank=gathered)
    elif args.mode == "ep_tier":
        # expert parallelism with every rank serving its own experts from tiers: half of them in GPU slots, the rest
        # through the host FFN
        from flyingfish_b200.parallel.ep import EPComm
        from flyingfish_b200.config import named_shape
        from flyingfish_b200.experts.provider import build_provider_from_weights
        spec = named_shape(args.model)
        ep = EPComm(dist.group.WORLD, device, spec.moe.num_experts, spec.hidden, max_rows=128, top_k=spec.moe.top_k)
        m = Model.load(args.model, Settings(capacity=256, max_batch=4, graph=False), device=device, seed=0, ep=ep)
        prov = build_provider_from_weights(m.engine.model, resident_fraction=0.5, threads=2, admission_cap=2)
        ep.provider = prov
        g = torch.Generator().manual_seed(100 + rank)
        prompt = torch.randint(0, 2048, (33,), generator=g).tolist()
        eng = m.engine
        prov.collect_freq = True
        seq = eng.add_sequence(prompt)
        first = eng.prefill([seq])[0]
        prov.collect_freq = False
        prov.begin_request()
        toks = [first] + [eng.decode([seq])[0] for _ in range(7)]
        gathered = [None] * world
        dist.all_gather_object(gathered, {"prompts": [prompt], "tokens": [toks], "res": dict(prov.res.stats),
                                          "prov": dict(prov.stats), "fp4": prov.fp4})
        torch.cuda.synchronize()
        ops.check_status(device)
        result.update(per_rank=gathered, stats=ep.stats)
    if rank == 0:
        Path(args.out).write_text(json.dumps(result))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
