"""Single-kernel timing harness (``python -m flyingfish_b200.utils.kbench <op> ...``).

Times one operator with CUDA events on the launching stream: warm-up iterations, then timed
iterations with an L2 flush (a write larger than L2) before each one unless the operands are
themselves larger than L2. Prints one JSON line per case with the achieved bandwidth / FLOP rate
and the fraction of the measured peaks of the box (``MEASURED_PEAKS.json`` at the repository root
when present, otherwise the stated fallback). The same harness feeds the calibration step and is
the command behind the ncu summaries under ``profiles/``.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from pathlib import Path

import torch

from .. import ops

ROOT = Path(__file__).resolve().parents[2]
L2_BYTES = 126 << 20


def peaks() -> dict:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class Flusher:
    def __init__(self, device):
        self.buf = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=device)

    def __call__(self):
        # several passes: the GPU must still be busy flushing when the timed launch is enqueued,
        # otherwise the host's launch latency lands between the two events
        for _ in range(4):
            self.buf.zero_()


def time_op(fn, iters: int, warmup: int, flush: Flusher | None, graph: bool = False) -> dict:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if graph:
        # an operator of several launches: replayed from a CUDA graph so that host time between its launches (Python,
        # allocator) does not sit inside the timed region, as in a captured decode step
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        fn = g.replay
    times = []
    for _ in range(iters):
        if flush is not None:
            flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3)      # us
    times.sort()
    # event timestamps tick in steps of about 2 us on some boxes: the mean over many iterations resolves finer
    return {"us_median": times[len(times) // 2], "us_min": times[0], "us_p90": times[int(len(times) * 0.9)],
            "us_mean": sum(times) / len(times)}


def bench_gemm(args) -> dict:
    dev = torch.device("cuda")
    m, n, k = args.m, args.n, args.k
    x = (torch.randn(m, k, device=dev) * 1.0).to(torch.bfloat16)
    w = (torch.randn(n, k, device=dev) * 0.05).to(torch.bfloat16)
    out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    byts = (m * k + n * k + m * n) * 2
    if args.torch:
        fn = lambda: torch.matmul(x, w.t(), out=out)
    elif getattr(args, "fp8", False):
        # block-scaled W8A8 linear: activation quantisation (1x128) + the tcgen05 FP8 GEMM, weights E4M3-resident
        from ..ops import quant_ops
        wq = quant_ops.Fp8Weight.from_dense(w)
        del w
        fn = lambda: ops.linear(x, wq, out=out)
        byts = m * k * 2 + wq.nbytes() + m * n * 2
    else:
        fn = lambda: ops.linear(x, w, out=out)
    r = time_op(fn, args.iters, args.warmup, Flusher(dev) if not args.no_flush else None, graph=getattr(args, "graph", False))
    pk = peaks()
    t = r["us_median"] * 1e-6
    r.update(op="gemm_torch" if args.torch else "gemm_fp8" if getattr(args, "fp8", False) else "gemm", m=m, n=n, k=k, gbs=byts / t / 1e9,
             tflops=2.0 * m * n * k / t / 1e12)
    r["frac_hbm"] = r["gbs"] / pk["hbm_gbs"]
    r["frac_tensor"] = r["tflops"] / pk["bf16_tflops"]
    r["peaks"] = pk["source"]
    return r


def bench_attn_decode(args) -> dict:
    dev = torch.device("cuda")
    b, ctx, hq, hkv, d = args.batch, args.ctx, args.hq, args.hkv, 128
    blocks_per = (ctx + 63) // 64
    nb = b * blocks_per
    kc = torch.randn(nb, hkv, 64, d, device=dev).to(torch.bfloat16)
    vc = torch.randn(nb, hkv, 64, d, device=dev).to(torch.bfloat16)
    bt = torch.arange(nb, dtype=torch.int32, device=dev).view(b, blocks_per)
    cl = torch.full((b,), ctx, dtype=torch.int32, device=dev)
    q = torch.randn(b, (hq + 2 * hkv) * d, device=dev).to(torch.bfloat16)
    fn = lambda: ops.attn_decode(q, kc, vc, bt, cl, hq, hkv, d, 1 / math.sqrt(d), max_ctx=ctx)
    if getattr(args, "torch", False):
        # the library arm: torch's fused attention over contiguous K / V of the same sizes (no paging, no packed Q)
        q4 = q[:, : hq * d].reshape(b, hq, 1, d).contiguous()
        k4 = kc.view(b, blocks_per, hkv, 64, d).permute(0, 2, 1, 3, 4).reshape(b, hkv, blocks_per * 64, d)[:, :, :ctx].contiguous()
        v4 = vc.view(b, blocks_per, hkv, 64, d).permute(0, 2, 1, 3, 4).reshape(b, hkv, blocks_per * 64, d)[:, :, :ctx].contiguous()
        fn = lambda: torch.nn.functional.scaled_dot_product_attention(q4, k4, v4, enable_gqa=True)
    byts = 2 * b * ctx * hkv * d * 2
    r = time_op(fn, args.iters, args.warmup, Flusher(dev) if not args.no_flush else None)
    pk = peaks()
    r.update(op="attn_decode", impl="torch_sdpa" if getattr(args, "torch", False) else "own", batch=b, ctx=ctx, hq=hq, hkv=hkv,
             gbs=byts / (r["us_median"] * 1e-6) / 1e9)
    r["frac_hbm"] = r["gbs"] / pk["hbm_gbs"]
    r["peaks"] = pk["source"]
    return r


def bench_attn_prefill(args) -> dict:
    dev = torch.device("cuda")
    b, ctx, hq, hkv, d = args.batch, args.ctx, args.hq, args.hkv, 128
    blocks_per = (ctx + 63) // 64
    nb = b * blocks_per
    kc = torch.randn(nb, hkv, 64, d, device=dev).to(torch.bfloat16)
    vc = torch.randn(nb, hkv, 64, d, device=dev).to(torch.bfloat16)
    bt = torch.arange(nb, dtype=torch.int32, device=dev).view(b, blocks_per)
    ql = torch.full((b,), ctx, dtype=torch.int32, device=dev)
    qs = (torch.arange(b, dtype=torch.int32, device=dev) * ctx)
    q = torch.randn(b * ctx, (hq + 2 * hkv) * d, device=dev).to(torch.bfloat16)
    fn = lambda: ops.attn_prefill(q, kc, vc, bt, qs, ql, ql, ctx, hq, hkv, d, 1 / math.sqrt(d))
    if getattr(args, "torch", False):
        q4 = q[:, : hq * d].reshape(b, ctx, hq, d).transpose(1, 2).contiguous()
        k4 = kc.view(b, blocks_per, hkv, 64, d).permute(0, 2, 1, 3, 4).reshape(b, hkv, blocks_per * 64, d)[:, :, :ctx].contiguous()
        v4 = vc.view(b, blocks_per, hkv, 64, d).permute(0, 2, 1, 3, 4).reshape(b, hkv, blocks_per * 64, d)[:, :, :ctx].contiguous()
        fn = lambda: torch.nn.functional.scaled_dot_product_attention(q4, k4, v4, is_causal=True, enable_gqa=True)
    flops = 4.0 * b * hq * d * ctx * (ctx + 1) / 2
    r = time_op(fn, args.iters, args.warmup, None)
    pk = peaks()
    r.update(op="attn_prefill", impl="torch_sdpa" if getattr(args, "torch", False) else "own", batch=b, ctx=ctx, hq=hq, hkv=hkv, tflops=flops / (r["us_median"] * 1e-6) / 1e12)
    r["frac_tensor"] = r["tflops"] / pk["bf16_tflops"]
    r["peaks"] = pk["source"]
    return r


def bench_moe(args) -> dict:
    """Routed experts of one MoE layer on one GPU (dispatch + gate/up GEMM with SwiGLU + down GEMM + combine), BF16
    expert stacks or packed NVFP4 stacks (``--fp4``; random codes: the timing does not depend on the values)."""
    from ..ops import moe_cuda, moe_ops
    dev = torch.device("cuda")
    rows, E, k, h, f = args.rows, args.experts, args.top_k, args.hidden, args.ffn
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(rows, h, generator=g, device=dev, dtype=torch.bfloat16) * 0.5
    gc = torch.Generator().manual_seed(2)
    ids = torch.stack([torch.randperm(E, generator=gc)[:k] for _ in range(rows)]).to(torch.int32).to(dev)
    wts = torch.softmax(torch.randn(rows, k, generator=gc), -1).to(dev)
    if args.fp4:
        rnd = lambda *shape: torch.randint(0, 256, shape, device=dev, dtype=torch.uint8)
        sc = lambda *shape: torch.randint(40, 60, shape, device=dev, dtype=torch.uint8)
        gs = torch.full((E,), 1e-3, device=dev)
        gu = moe_cuda.Nvfp4Experts(rnd(E, 2 * f, h // 2), sc(E, 2 * f, h // 16), gs, gate_up=True)
        dn = moe_cuda.Nvfp4Experts(rnd(E, h, f // 2), sc(E, h, f // 16), gs)
        fn = lambda: moe_cuda.experts_forward_nvfp4(x, wts, ids, gu, dn)
        byts = gu.nbytes() + dn.nbytes()
    elif getattr(args, "fp8", False):
        # FP8-resident experts (E4M3 codes + 128x128 scales; random codes: the timing does not depend on the values)
        from ..ops import quant_ops
        codes = lambda *shape: torch.randint(0, 120, shape, device=dev, dtype=torch.uint8)
        sc = lambda *shape: torch.full(shape, 1e-2, device=dev, dtype=torch.float32)
        gu = quant_ops.Fp8Experts(codes(E, 2 * f, h), sc(E, (2 * f + 127) // 128, h // 128), interleaved=True)
        dn = quant_ops.Fp8Experts(codes(E, h, f), sc(E, (h + 127) // 128, f // 128), interleaved=False)
        fn = lambda: quant_ops.experts_forward_fp8(x, wts, ids, gu, dn)
        byts = E * 3 * f * h
    else:
        wgu = torch.randn(E, 2 * f, h, generator=g, device=dev, dtype=torch.bfloat16) * 0.02
        wd = torch.randn(E, h, f, generator=g, device=dev, dtype=torch.bfloat16) * 0.02
        fn = lambda: moe_ops.experts_forward(x, wts, ids, wgu, wd, 0)
        byts = (wgu.numel() + wd.numel()) * 2
    r = time_op(fn, args.iters, args.warmup, Flusher(dev) if not args.no_flush else None, graph=getattr(args, "graph", False))
    pk = peaks()
    t = r["us_mean"] * 1e-6
    r.update(op="moe_fp4" if args.fp4 else "moe_fp8" if getattr(args, "fp8", False) else "moe", rows=rows, experts=E, top_k=k, hidden=h, ffn=f, expert_bytes=byts,
             gbs=byts / t / 1e9, tflops=2.0 * rows * k * 3 * f * h / t / 1e12)
    r["frac_hbm"] = r["gbs"] / pk["hbm_gbs"]
    r["peaks"] = pk["source"]
    return r


def bench_attn_mixed(args) -> dict:
    """Decode attention over the affine8 cache (sink + sealed 8-bit groups + ``--recent`` BF16 tokens) against the same
    contexts held entirely in BF16 pages."""
    from ..engine.kv_cache import PagedKVCache
    from ..engine.kv_compact import CompactKV
    dev = torch.device("cuda")
    b, ctx, hq, hkv, d = args.batch, args.ctx, args.hq, args.hkv, 128
    per = (ctx + 63) // 64
    kv = PagedKVCache(1, hkv, d, b * per + 1, 64, torch.bfloat16, dev)
    kv.k[0].normal_(); kv.v[0].normal_()
    q = torch.randn(b, (hq + 2 * hkv) * d, device=dev).to(torch.bfloat16)
    cl = torch.full((b,), ctx, dtype=torch.int32, device=dev)
    for i in range(b):
        kv.add_sequence(i); kv.reserve(i, ctx); kv.commit(i, ctx)
    bt_full = torch.tensor([kv.seqs[i].blocks for i in range(b)], dtype=torch.int32, device=dev)
    flush = Flusher(dev) if not args.no_flush else None
    plain = time_op(lambda: ops.attn_decode(q, kv.k[0], kv.v[0], bt_full, cl, hq, hkv, d, 1 / math.sqrt(d), max_ctx=ctx),
                    args.iters, args.warmup, flush)
    c = CompactKV(1, hkv, d, b * (ctx // 128) + 1, dev, recent=args.recent)
    kv.compact = c
    for i in range(b):
        c.seal(kv, i)
    mg = max(ctx // 128, 1)
    bt = torch.tensor([[x if x >= 0 else 0 for x in kv.seqs[i].blocks] for i in range(b)], dtype=torch.int32, device=dev)
    gt = torch.tensor([c.groups[i] + [0] * (mg - len(c.groups[i])) for i in range(b)], dtype=torch.int32, device=dev)
    ks = torch.tensor([c.sealed_tokens(i) for i in range(b)], dtype=torch.int32, device=dev)
    mixed = time_op(lambda: ops.attn_decode_mixed(q, kv.k[0], kv.v[0], c, 0, bt, cl, ks, gt, hq, hkv, d, 1 / math.sqrt(d),
                                                  max_ctx=ctx), args.iters, args.warmup, flush)
    sealed = int(ks[0])
    bytes_bf16 = 2 * b * ctx * hkv * d * 2
    bytes_mixed = 2 * b * hkv * ((ctx - sealed + 64) * d * 2 + (sealed - 64) * d) + b * hkv * (sealed // 128) * (d * 8 + 128 * 8)
    return {"op": "attn_mixed", "batch": b, "ctx": ctx, "recent": args.recent, "sealed_tokens": sealed,
            "bf16_us": plain["us_median"], "mixed_us": mixed["us_median"], "bf16_bytes": bytes_bf16, "mixed_bytes": bytes_mixed,
            "bf16_gbs": bytes_bf16 / plain["us_median"] / 1e3, "mixed_gbs": bytes_mixed / mixed["us_median"] / 1e3}


def bench_gdn(args) -> dict:
    """Gated delta rule over packed prefill rows: the token-by-token kernel against the chunked tensor-core form."""
    from ..ops import gdn_ops
    dev = torch.device("cuda")
    b, n, heads = args.batch, args.ctx, args.hq
    rows = b * n
    q = torch.randn(rows, heads, 128, device=dev); k = torch.randn(rows, heads, 128, device=dev)
    q = q / q.norm(dim=-1, keepdim=True) * 128 ** -0.5
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(rows, heads, 128, device=dev)
    beta = torch.sigmoid(torch.randn(rows, heads, device=dev)); dec = -torch.rand(rows, heads, device=dev) * 0.3
    state = torch.zeros(b, heads, 128, 128, device=dev)
    rs = (torch.arange(b + 1, dtype=torch.int32, device=dev) * n)
    slots = torch.arange(b, dtype=torch.int32, device=dev)
    flush = Flusher(dev) if not args.no_flush else None
    rec = time_op(lambda: gdn_ops.recurrent_slots(q, k, v, beta, dec, state, rs, slots), args.iters, args.warmup, flush)
    state.zero_()
    chk = time_op(lambda: gdn_ops.chunked_slots(q, k, v, beta, dec, state, rs, slots), args.iters, args.warmup, flush)
    return {"op": "gdn", "sequences": b, "tokens": n, "heads": heads, "recurrent_us": rec["us_median"],
            "chunked_us": chk["us_median"], "speedup": rec["us_median"] / chk["us_median"],
            "chunked_us_per_chunk": chk["us_median"] / max(n // 64, 1)}


def bench_speech(args) -> dict:
    """Speech recognition at the published Parakeet-TDT geometry (random weights): log-mel, encoder and greedy
    transducer decode of ``--batch`` utterances of ``--seconds`` each, and the relative-position attention kernel of one
    layer alone with a library soft-max attention of the same shape (no position term) beside it."""
    from ..ops import speech_ops
    from ..speech import ParakeetModel, ParakeetSpec
    dev = torch.device("cuda")
    spec = ParakeetSpec()
    if args.attention_only:
        t, h, d = spec.encoder.sub_len(int(args.seconds * 100)), spec.encoder.heads, spec.encoder.head_dim
        qkv = torch.randn(args.batch * t, 3 * h * d, device=dev).to(torch.bfloat16)
        pos = torch.randn(2 * t - 1, h * d, device=dev).to(torch.bfloat16)
        u, v = torch.randn(h, d, device=dev), torch.randn(h, d, device=dev)
        lens = torch.full((args.batch,), t, dtype=torch.int32, device=dev)
        hd = h * d
        att = time_op(lambda: speech_ops.relpos_attention(qkv[:, :hd], qkv[:, hd:2 * hd], qkv[:, 2 * hd:], pos, u, v, lens,
                                                          args.batch, h), args.iters, args.warmup, None)
        flops = 3 * 2.0 * args.batch * h * t * t * d
        return {"op": "relpos_attention", "batch": args.batch, "rows": t, "heads": h, "head_dim": d, "us": att["us_median"],
                "tflops": flops / att["us_median"] / 1e6}
    model = ParakeetModel.random(spec, dev, seed=0, max_batch=min(args.batch, 32))
    g = torch.Generator().manual_seed(0)
    waves = [0.1 * torch.randn(int(args.seconds * 16000), generator=g) for _ in range(args.batch)]
    audio_s = args.seconds * args.batch

    def front():
        return model.mel.extract(waves)

    feat, valid = front()
    vl = valid.tolist()
    mel = time_op(front, args.iters, args.warmup, None)
    enc = time_op(lambda: model.encoder.encode(feat, vl), args.iters, args.warmup, None)
    encoded, rows = model.encoder.encode(feat, vl)
    nb = min(args.batch, model.decoder.max_batch)
    projs = [model.decoder.project(encoded[b]) for b in range(nb)]
    model.decoder.decode_batch(projs, rows[:nb])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    traj = model.decoder.decode_batch(projs, rows[:nb])[0]
    e1.record()
    torch.cuda.synchronize()
    dec_ms = e0.elapsed_time(e1) / nb                       # the utterances of a batch step together
    t, h, d = encoded.shape[1], spec.encoder.heads, spec.encoder.head_dim
    qkv = torch.randn(args.batch * t, 3 * h * d, device=dev).to(torch.bfloat16)
    pos = torch.randn(2 * t - 1, h * d, device=dev).to(torch.bfloat16)
    u, v = torch.randn(h, d, device=dev), torch.randn(h, d, device=dev)
    lens = torch.tensor(rows, dtype=torch.int32, device=dev)
    hd = h * d
    att = time_op(lambda: speech_ops.relpos_attention(qkv[:, :hd], qkv[:, hd:2 * hd], qkv[:, 2 * hd:], pos, u, v, lens,
                                                      args.batch, h), args.iters, args.warmup, None)
    q4 = qkv.reshape(args.batch, t, 3, h, d).permute(2, 0, 3, 1, 4).contiguous()
    lib = time_op(lambda: torch.nn.functional.scaled_dot_product_attention(q4[0], q4[1], q4[2]), args.iters, args.warmup, None)
    flops = 3 * 2.0 * args.batch * h * t * t * d                  # content, position and PV products
    total_ms = (mel["us_median"] + enc["us_median"]) / 1e3 + dec_ms * args.batch
    return {"op": "speech", "batch": args.batch, "seconds": args.seconds, "encoder_rows": t,
            "logmel_us": mel["us_median"], "encoder_ms": enc["us_median"] / 1e3, "decode_ms_per_utterance": dec_ms,
            "decode_steps": traj.steps, "decode_state_reads": traj.state_reads, "decode_us_per_step": dec_ms * 1e3 / max(traj.steps, 1),
            "audio_seconds_per_second_encoder": audio_s / (enc["us_median"] / 1e6),
            "audio_seconds_per_second_total": audio_s / (total_ms / 1e3),
            "relpos_attention_us": att["us_median"], "relpos_attention_tflops": flops / att["us_median"] / 1e6,
            "library_sdpa_no_position_term_us": lib["us_median"]}


def bench_diarize(args) -> dict:
    """Speaker diarization at the published geometry (31 layers, hidden 512, 8 heads of 64, random weights): one full
    offline window (speaker cache + FIFO + chunk + look-ahead = 684 rows) through encoder and head, one low-latency
    streaming window (264 + 264 + 9 + 4 rows), and a whole clip of ``--seconds`` through the offline chunking with the
    cache policy on the host."""
    from ..speech import diarization as dz
    dev = torch.device("cuda")
    spec = dz.DiarizationSpec()
    model = dz.DiarizationModel.random(spec, dev, seed=0)
    out = {"op": "diarize", "seconds": args.seconds}
    for name, rows in (("offline_window", spec.max_encoder_rows()), ("stream_window", spec.cache.frames + spec.cache.fifo + 13)):
        emb = (torch.randn(rows, spec.hidden, device=dev) * 0.5).to(torch.bfloat16)
        t = time_op(lambda: model.classify(model.encode(emb, rows)), args.iters, args.warmup, None)
        flops = spec.layers * (2.0 * rows * spec.hidden * (4 * spec.hidden + 2 * spec.intermediate) + 4.0 * rows * rows * spec.hidden)
        out[name] = {"rows": rows, "us": t["us_median"], "tflops": flops / t["us_median"] / 1e6}
    frames = int(args.seconds * 100)
    feat = torch.randn(frames, spec.mel.mel_bins, device=dev)
    model.offline(feat)                                            # warm-up
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    calls = model.encoder_calls
    model.offline(feat)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    out.update({"clip_ms": ms, "clip_windows": model.encoder_calls - calls, "audio_seconds_per_second": args.seconds / (ms / 1e3),
                "cache_compressions": model.last_state.updates})
    return out


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(prog="kbench")
    sub = ap.add_subparsers(dest="op", required=True)
    for name in ("gemm", "attn_decode", "attn_prefill", "attn_mixed", "gdn", "moe", "speech", "diarize"):
        p = sub.add_parser(name)
        p.add_argument("--iters", type=int, default=20)
        p.add_argument("--warmup", type=int, default=3)
        p.add_argument("--no-flush", action="store_true")
        if name == "gemm":
            p.add_argument("--m", type=int, default=64)
            p.add_argument("--n", type=int, default=4096)
            p.add_argument("--k", type=int, default=4096)
            p.add_argument("--torch", action="store_true", help="time torch.matmul (cuBLAS) instead, as the baseline")
            p.add_argument("--fp8", action="store_true", help="FP8-resident weight (E4M3, 128x128 scales), W8A8 kernel")
            p.add_argument("--graph", action="store_true", help="replay the operator from a CUDA graph (no host gaps)")
        elif name == "speech":
            p.add_argument("--batch", type=int, default=8)
            p.add_argument("--seconds", type=float, default=30.0)
            p.add_argument("--attention-only", action="store_true", help="only the relative-position attention kernel of one layer")
        elif name == "diarize":
            p.add_argument("--seconds", type=float, default=120.0)
        elif name == "moe":
            p.add_argument("--rows", type=int, default=128)
            p.add_argument("--experts", type=int, default=128)
            p.add_argument("--top-k", type=int, default=8)
            p.add_argument("--hidden", type=int, default=4096)
            p.add_argument("--ffn", type=int, default=1536)
            p.add_argument("--fp4", action="store_true", help="packed NVFP4 expert stacks expanded inside the GEMM")
            p.add_argument("--fp8", action="store_true", help="FP8-resident expert stacks (E4M3, 128x128 scales), W8A8 grouped GEMMs")
            p.add_argument("--graph", action="store_true", help="replay the operator from a CUDA graph (no host gaps)")
        else:
            p.add_argument("--batch", type=int, default=64)
            p.add_argument("--ctx", type=int, default=1024)
            p.add_argument("--hq", type=int, default=32)
            p.add_argument("--hkv", type=int, default=8)
            if name == "attn_mixed":
                p.add_argument("--recent", type=int, default=2048)
            if name in ("attn_decode", "attn_prefill"):
                p.add_argument("--torch", action="store_true", help="time torch's fused attention on contiguous K / V instead")
    args = ap.parse_args(argv)
    fn = {"gemm": bench_gemm, "attn_decode": bench_attn_decode, "attn_prefill": bench_attn_prefill, "attn_mixed": bench_attn_mixed, "gdn": bench_gdn,
          "moe": bench_moe, "speech": bench_speech, "diarize": bench_diarize}[args.op]
    print(json.dumps(fn(args)))
    ops.check_status()


if __name__ == "__main__":
    main(sys.argv[1:])
