"""Device timeline: where the time of a step goes *inside* and *between* kernels.

With ``FLYINGFISH_TIMELINE=1`` the tracing build of the kernel library is loaded
(``ops/build.py`` ``timeline=True``, ``-DFF_TIMELINE``). One thread per CTA then stamps
``%globaltimer`` at the phases of interest (entry, after the programmatic-dependency wait, first
data, last MMA, epilogue, exit ...) into the enlarged status buffer. This module reads the records
back and prints, per kernel launch, when its CTAs started relative to the end of the previous
launch and how long each phase took. It is the tool for questions ``ncu`` cannot answer: launch
gaps, overlap obtained from programmatic dependent launch, pipeline fill time of one kernel inside
a real decode step.

Usage::

    FLYINGFISH_TIMELINE=1 python -m flyingfish_b200.utils.timeline --model llama3-8b-shape --batch 64 --ctx 1024

The reference's counterpart is its host-side stage timing (src/model.rs ``decode_stage_ms``) which
needs a device synchronise per stage; stamps taken on the device do not perturb the step.
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

KERNEL_NAMES = {1: "gemm_bf16", 2: "gemm_skinny", 3: "embed", 4: "norm", 5: "rope_kv", 6: "act", 7: "attn_decode",
                8: "attn_prefill", 9: "sample", 10: "allreduce", 11: "gemm_ar", 30: "chain"}


def reset(device=None) -> None:
    from ..ops import lib
    assert lib.TIMELINE, "set FLYINGFISH_TIMELINE=1 before importing the package"
    lib.status_tensor(device)[8:16].zero_()


def read(device=None) -> np.ndarray:
    """Records sorted by time: structured array (t_ns, kid, phase, sm, block)."""
    from ..ops import lib
    assert lib.TIMELINE, "set FLYINGFISH_TIMELINE=1 before importing the package"
    torch.cuda.synchronize()
    st = lib.status_tensor(device)
    n = min(int(st[8].item()), lib.TIMELINE_CAP)
    raw = st[16: 16 + 4 * n].cpu().numpy().reshape(n, 4)
    out = np.zeros(n, dtype=[("t", np.int64), ("kid", np.int32), ("phase", np.int32), ("sm", np.int32), ("block", np.int32)])
    out["t"] = raw[:, 0].astype(np.uint32).astype(np.int64) | (raw[:, 1].astype(np.uint32).astype(np.int64) << 32)
    out["kid"] = raw[:, 2] >> 16
    out["phase"] = raw[:, 2] & 0xFFFF
    out["sm"] = (raw[:, 3].astype(np.uint32) >> 20).astype(np.int32)
    out["block"] = raw[:, 3] & 0xFFFFF
    return np.sort(out, order="t")


def split_launches(rec: np.ndarray, slack_ns: int = 1500) -> list[np.ndarray]:
    """Group records into launches. A launch of a kernel starts at the phase-0 stamp of its block 0;
    a CTA belongs to the launch whose block 0 started last before the CTA's own phase-0 stamp (CTAs
    of one launch start within ``slack_ns`` of each other's dispatch order), and the later stamps of
    that CTA follow it. Launches come back ordered by start time."""
    groups: dict[tuple[int, int], list[int]] = {}
    out: dict[tuple[int, int], list[int]] = {}
    for kid in np.unique(rec["kid"]):
        idx = np.nonzero(rec["kid"] == kid)[0]
        sub = rec[idx]
        starts = sub["t"][(sub["phase"] == 0) & (sub["block"] == 0)]
        if len(starts) == 0:
            continue
        cur: dict[int, int] = {}
        for i, r in zip(idx, sub):
            b = int(r["block"])
            if r["phase"] == 0:
                cur[b] = max(int(np.searchsorted(starts - slack_ns, r["t"], side="right")) - 1, 0)
            if b in cur:
                out.setdefault((int(kid), cur[b]), []).append(int(i))
    launches = [rec[np.array(ix, dtype=np.int64)] for ix in out.values()]
    launches.sort(key=lambda la: int(la["t"][(la["phase"] == 0)].min()) if (la["phase"] == 0).any() else int(la["t"].min()))
    return launches


def summarise(rec: np.ndarray, limit: int = 60) -> list[dict]:
    rows = []
    prev_end = None
    for la in split_launches(rec)[:limit]:
        kid = int(la["kid"][0])
        t0 = int(la["t"].min())
        row = {"kernel": KERNEL_NAMES.get(kid, str(kid)), "ctas": int((la["phase"] == 0).sum()),
               "gap_us": None if prev_end is None else round((t0 - prev_end) / 1e3, 2),
               "span_us": round((int(la["t"].max()) - t0) / 1e3, 2)}
        for ph in sorted(set(la["phase"].tolist())):
            v = (la["t"][la["phase"] == ph] - t0) / 1e3
            row[f"p{ph}"] = [round(float(v.min()), 2), round(float(np.median(v)), 2), round(float(v.max()), 2)]
        rows.append(row)
        prev_end = int(la["t"].max())
    return rows


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="llama3-8b-shape")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--ctx", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--layers", type=int, default=0, help="truncate the model to this many layers (0 = all)")
    ap.add_argument("--limit", type=int, default=40)
    ap.add_argument("--no-graph", action="store_true")
    args = ap.parse_args()
    import dataclasses

    from ..config import Settings, named_shape
    from ..engine.engine import Engine
    from ..models.decoder import DecoderModel
    from ..models.weights import random_decoder_weights
    from ..planner.plan import plan_engine
    spec = named_shape(args.model)
    if args.layers:
        spec = dataclasses.replace(spec, layers=args.layers)
    dev = torch.device("cuda", 0)
    settings = Settings(capacity=((args.ctx + 64 + 63) // 64) * 64, max_batch=args.batch, graph=not args.no_graph)
    weights = random_decoder_weights(spec, 0, dev)
    plan = plan_engine(spec, settings, dev, weights_bytes=weights.nbytes(), tp=1)
    eng = Engine(DecoderModel(weights), spec, settings, plan.kv_blocks, dev, max_prefill_rows=plan.prefill_chunk)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, spec.vocab, (args.ctx,), generator=g).tolist() for _ in range(args.batch)]
    seqs = [eng.add_sequence(p) for p in prompts]
    eng.prefill(seqs)
    for _ in range(args.steps):
        eng.decode(seqs)
    reset(dev)
    eng.decode(seqs)
    rec = read(dev)
    for row in summarise(rec, args.limit):
        print(json.dumps(row))


if __name__ == "__main__":
    main()
