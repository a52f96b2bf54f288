"""``ff`` command line (``python -m flyingfish_b200.cli`` / the ``ff`` console script).

Same shape as the reference's CLI (src/main.rs:19-60, 177-516): global options come BEFORE the
subcommand (``ff --model M generate --prompt ...``), ``--model`` falls back to
``FLYINGFISH_MODEL``, results are one JSON object on stdout, decisions are JSON lines on stderr.
Subcommands: calibrate, generate, serve, bench, profile, inspect, tokenize, embed, verify,
compare-prefill, compare-log, plus the speculative-decoding tools (verify-spec, bench-spec,
profile-spec for MTP; replay-draft, replay-tree, check-tree-greedy, compare-tree-builders,
compare-tree-padding, compare-spec-graph for a draft model). ``--model`` accepts a checkpoint directory or one of the named random-init shapes
(``ff inspect --shapes`` lists them).

Writes never go inside a model directory or under a path component named ``models`` and never
overwrite an existing file (src/main.rs:518-545).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time
from pathlib import Path

from .config import NAMED_SHAPES, Settings


DSPARK_TOOLS = ("replay-draft", "replay-tree", "check-tree-greedy", "compare-tree-builders", "compare-tree-padding",
                "compare-spec-graph")


def _global_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="ff", description="flyingfish_b200 inference engine")
    p.add_argument("--model", default=os.environ.get("FLYINGFISH_MODEL"))
    p.add_argument("--draft-model", default=os.environ.get("FLYINGFISH_DRAFT_MODEL"))
    p.add_argument("--device", type=int, default=0)
    p.add_argument("--verbose", action="store_true")
    p.add_argument("--capacity", type=int, default=4096)
    p.add_argument("--chunk", type=int, default=None)
    p.add_argument("--device-budget-gib", type=float, default=None)
    p.add_argument("--tree-builder", choices=["waves", "serial", "markov"], default="waves")
    p.add_argument("--spec-budget", choices=["chain", "tree16", "tree32", "tree64"], default="chain")
    p.add_argument("--spec-graph", type=lambda s: s.lower() != "false", default=True)
    p.add_argument("--prefix-cache", type=lambda s: s.lower() == "true", default=False)
    p.add_argument("--kv-format", choices=["bf16", "affine8"], default="bf16")
    p.add_argument("--kv-recent", type=int, default=2048, help="affine8: newest tokens kept in BF16 (older 128-token groups are sealed)")
    p.add_argument("--runtime-dir", default=os.environ.get("FLYINGFISH_RUNTIME_DIR"))
    p.add_argument("--dram-gb-s", type=float, default=6550.0)
    p.add_argument("--gemm-tflops", type=float, default=1385.0)
    p.add_argument("--max-batch", type=int, default=64)
    p.add_argument("--tp", type=int, default=1, help="tensor-parallel ranks (the command re-launches itself, one process per GPU)")
    p.add_argument("--cpu", action="store_true", help="run on the host (tiny shapes / debugging)")
    p.add_argument("--seed", type=int, default=0)
    sub = p.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate")
    src = g.add_mutually_exclusive_group(required=True)
    src.add_argument("--prompt")
    src.add_argument("--tokens")
    src.add_argument("--tokens-file")
    g.add_argument("--max-new-tokens", type=int, default=32)
    g.add_argument("--graph", action="store_true")
    g.add_argument("--mtp", type=int, default=None, choices=range(0, 5))
    g.add_argument("--dump")
    g.add_argument("--trace-layer", type=int, default=None)
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--diffusion-steps", type=int, default=0,
                   help="masked-diffusion models: number of denoising passes (default: one per 4 new tokens)")
    g.add_argument("--diffusion-block", type=int, default=0, help="denoise the canvas in blocks of this many tokens")
    g.add_argument("--image", action="append", default=[],
                   help="PNG file for each image placeholder of the prompt (vision-language models)")

    s = sub.add_parser("serve")
    s.add_argument("--port", type=int, default=8080)
    s.add_argument("--mtp", type=int, default=None, choices=range(0, 5))
    s.add_argument("--allow-sampling", action="store_true")

    b = sub.add_parser("bench")
    b.add_argument("--steps", type=int, default=256)
    b.add_argument("--warmup", type=int, default=32)
    b.add_argument("--runs", type=int, default=3)
    b.add_argument("--graph", action="store_true")
    b.add_argument("--batch", type=int, default=1)
    b.add_argument("--prompt-tokens", type=int, default=128)

    pr = sub.add_parser("profile")
    pr.add_argument("--phase", choices=["decode", "prefill"], default="decode")
    pr.add_argument("--prompt-tokens", type=int, default=128)

    i = sub.add_parser("inspect")
    i.add_argument("--shapes", action="store_true")

    t = sub.add_parser("tokenize")
    t.add_argument("--prompt", required=True)

    c = sub.add_parser("calibrate")
    c.add_argument("--force", action="store_true")

    e = sub.add_parser("embed")
    e.add_argument("--prompt", required=True)

    v = sub.add_parser("verify")
    v.add_argument("--trace", required=True)
    v.add_argument("--reference", required=True)
    v.add_argument("--limits")
    cp = sub.add_parser("compare-prefill")
    cp.add_argument("--trace", required=True)
    cp.add_argument("--reference", required=True)
    cl = sub.add_parser("compare-log")
    cl.add_argument("--a", required=True)
    cl.add_argument("--b", required=True)

    tr = sub.add_parser("transcribe")
    tr.add_argument("input", help="RIFF/WAVE file (any rate and channel count; mixed down and resampled to 16 kHz)")
    tr.add_argument("--format", choices=["txt", "json", "srt", "vtt"], default="txt")
    tr.add_argument("--output", help="file to write instead of standard output")
    tr.add_argument("--stream", action="store_true")
    tr.add_argument("--source-lang", default="en")
    tr.add_argument("--target-lang", default="en")
    tr.add_argument("--no-pnc", action="store_true", help="Canary: no punctuation and capitalisation")
    tr.add_argument("--diarization-model", help="multitalker archives: diarization checkpoint whose speaker activity selects the lanes")
    tr.add_argument("--masked-asr", action="store_true", help="multitalker archives: mask each lane's log-mel input instead of conditioning layer 0")

    dz = sub.add_parser("diarize")
    dz.add_argument("input", help="RIFF/WAVE file (mixed down and resampled to the model's rate)")
    dz.add_argument("--format", choices=["rttm", "json"], default="rttm")
    dz.add_argument("--output", help="file to write instead of standard output")
    dz.add_argument("--stream", action="store_true", help="chunk-wise with look-ahead, as live audio would arrive")
    dz.add_argument("--mode", help="streaming latency mode named in the processor configuration")
    dz.add_argument("--threshold", type=float, default=0.5, help="speaker activity probability that counts as speech")

    t3 = sub.add_parser("to-3d")
    t3.add_argument("input", help="safetensors file with the shape decoder's output: `coords` [n, 4] int32 and either `fields` [n, 7] "
                                  "(dual grid), or `scalar` [c] on the cubes' shared corners (lexicographic corner order), or "
                                  "`cubes` [n, 8], `positions` [c, 3], `scalar` [c] (explicit corner field)")
    t3.add_argument("--output", required=True, help="mesh file to write (.ply or .obj)")
    t3.add_argument("--resolution", type=int, default=0, help="grid side of the dual-grid fields")
    t3.add_argument("--min-component", type=float, default=0.0, help="drop components below this share of the faces")
    t3.add_argument("--fill-holes", type=int, default=0, help="close boundary loops of at most this many edges")
    t3.add_argument("--faces", type=int, default=0, help="simplify to at most this many faces")
    t3.add_argument("--unit-ball", action="store_true", help="centre the mesh and scale it into the unit ball")

    for name in DSPARK_TOOLS:
        dp = sub.add_parser(name)
        dp.add_argument("--prompt-tokens", type=int, default=48)
        dp.add_argument("--max-new-tokens", type=int, default=24)
        dp.add_argument("--trace", help="replay tools: trace file to write (first run) or to reproduce (later runs)")
        dp.add_argument("--strict", action="store_true")

    for name in ("verify-spec", "bench-spec", "profile-spec"):
        sp = sub.add_parser(name)
        sp.add_argument("--prompt-tokens", type=int, default=64)
        sp.add_argument("--max-new-tokens", type=int, default=64)
        sp.add_argument("--mtp", type=int, default=2)
        sp.add_argument("--strict", action="store_true")
    return p


def parse_tokens_arg(args) -> list[int] | None:
    """``--tokens a,b,c`` or ``--tokens-file`` holding an array, ``{"input_ids": [...]}`` or a nested
    first row (src/main.rs:73-97)."""
    if getattr(args, "tokens", None):
        return [int(x) for x in args.tokens.split(",") if x.strip()]
    if getattr(args, "tokens_file", None):
        data = json.loads(Path(args.tokens_file).read_text())
        if isinstance(data, dict):
            data = data["input_ids"]
        if data and isinstance(data[0], list):
            data = data[0]
        return [int(x) for x in data]
    return None


def check_output_path(path: str | Path, model: str | None) -> Path:
    p = Path(path).resolve()
    if p.exists():
        raise SystemExit(f"refusing to overwrite {p}")
    if any(part == "models" for part in p.parts):
        raise SystemExit(f"refusing to write under a 'models' directory: {p}")
    if model and Path(model).is_dir():
        m = Path(model).resolve()
        if m == p or m in p.parents:
            raise SystemExit(f"refusing to write inside the model directory: {p}")
    return p


def settings_from(args) -> Settings:
    return Settings(device=args.device, capacity=args.capacity, chunk=args.chunk,
                    device_budget_gib=args.device_budget_gib, draft_model=args.draft_model,
                    tree_builder=args.tree_builder,
                    spec_budget=args.spec_budget if args.draft_model else "chain",
                    spec_graph=args.spec_graph, prefix_cache=args.prefix_cache, kv_format=args.kv_format, kv_recent=args.kv_recent,
                    runtime_dir=args.runtime_dir, dram_gb_s=args.dram_gb_s, gemm_tflops=args.gemm_tflops,
                    verbose=args.verbose, max_batch=args.max_batch, tp=args.tp)


def resolve_mtp_depth(requested: int | None, has_mtp: bool, arch: str) -> int:
    """Default depth 4 when the checkpoint ships MTP tensors and the architecture binds them,
    0 for DeepSeek-style checkpoints unless asked for (src/main.rs:771-809)."""
    if requested is not None:
        if requested > 0 and not has_mtp:
            raise SystemExit("--mtp given but the checkpoint has no MTP component")
        return requested
    if not has_mtp:
        return 0
    return 0 if arch == "deepseek_v3" else 4


def check_flags(args) -> None:
    """Every flag either changes behaviour or is refused: nothing is parsed and then ignored."""
    if args.kv_format != "bf16":
        # the sealed 8-bit store is read by plain decode steps only
        if args.draft_model or args.prefix_cache or args.command in DSPARK_TOOLS + ("verify-spec", "bench-spec", "profile-spec") \
                or (args.command == "serve" and getattr(args, "mtp", None) not in (None, 0)):
            raise SystemExit("--kv-format affine8 does not combine with speculative decoding or the prefix cache "
                             "(verification rows and shared prefixes read BF16 pages)")
    if args.tp < 1 or (args.tp > 1 and args.cpu):
        raise SystemExit("--tp needs one CUDA device per rank")
    if args.command in ("transcribe", "diarize", "to-3d") and (args.draft_model or args.prefix_cache or args.kv_format != "bf16"):
        raise SystemExit(f"{args.command} takes none of the text-generation flags")
    if args.tp > 1 and args.command not in ("generate", "bench", "serve"):
        raise SystemExit(f"--tp applies to generate, bench and serve, not to {args.command}")
    if args.command in DSPARK_TOOLS and not args.draft_model:
        raise SystemExit(f"{args.command} needs --draft-model")
    if args.draft_model and args.command != "generate" and args.command not in DSPARK_TOOLS:
        raise SystemExit("--draft-model applies to generate and the draft-model tools")
    if args.draft_model and args.tp > 1:
        raise SystemExit("--draft-model with --tp is not supported")
    if args.command in ("check-tree-greedy", "replay-tree", "compare-tree-builders") and args.spec_budget == "chain":
        args.spec_budget = "tree16"
    if args.spec_budget != "chain" and not args.draft_model:
        raise SystemExit("--spec-budget needs --draft-model")
    if args.prefix_cache and args.command != "generate":
        raise SystemExit("--prefix-cache applies to generate (the server's batched scheduler does not consult the store)")
    if not args.spec_graph and not args.draft_model:
        raise SystemExit("--spec-graph applies to --draft-model speculation")
    if args.prefix_cache and args.tp > 1:
        raise SystemExit("--prefix-cache with --tp is not supported")


def _world() -> tuple[int, int, int]:
    return int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))


def relaunch_tp(args, argv: list[str]) -> int | None:
    """``--tp N`` outside a launcher: start N ranks of this same command line (rank 0 prints the result)."""
    if args.tp <= 1 or _world()[0] > 1:
        return None
    import subprocess
    port = int(os.environ.get("FLYINGFISH_MASTER_PORT", "29517"))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.tp}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "flyingfish_b200.cli", *argv]
    return subprocess.call(cmd)


def _load(args):
    import torch
    from .api import Model
    from .utils.log import with_verbose
    if not args.model:
        raise SystemExit("--model (or FLYINGFISH_MODEL) is required before the subcommand")
    st = settings_from(args)
    world, rank, local = _world()
    comm = None
    if args.tp > 1:
        if world != args.tp:
            raise SystemExit(f"--tp {args.tp} but the launcher started {world} ranks")
        import torch.distributed as dist
        from .parallel.comm import TPComm
        from .config import named_shape, read_model_spec
        torch.cuda.set_device(local)
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        spec = read_model_spec(args.model) if Path(args.model).is_dir() else named_shape(args.model)
        comm = TPComm.create(dist.group.WORLD, torch.device("cuda", local), slot_bytes=(8192 // world) * spec.hidden * 2)
        device = f"cuda:{local}"
        st.device = local
    else:
        device = "cpu" if args.cpu or not torch.cuda.is_available() else f"cuda:{args.device}"
    with with_verbose(args.verbose):
        return Model.load(args.model, st, device=device, seed=args.seed, comm=comm)


def cmd_generate(args) -> dict:
    from .api import generate_plain
    from .loaders.tokenizer import ByteTokenizer
    if args.dump and args.graph:
        raise SystemExit("--dump is incompatible with --graph")
    if args.dump:
        check_output_path(args.dump, args.model)
    model = _load(args)
    tk = model.tokenizer or ByteTokenizer(model.spec.vocab)
    ids = parse_tokens_arg(args)
    if ids is None:
        ids = tk.encode(args.prompt)
    if len(ids) + args.max_new_tokens > args.capacity:
        raise SystemExit(f"prompt ({len(ids)}) + max-new-tokens ({args.max_new_tokens}) exceeds --capacity {args.capacity}")
    trace = None
    if args.dump:
        from .utils.trace import Trace
        trace = Trace(device=str(model.engine.device), only_layer=args.trace_layer)
        model.engine.model.trace = trace
    if model.spec.arch == "diffusion_lm":
        from .spec.diffusion import DiffusionTrace, diffusion_generate
        tr = DiffusionTrace()
        steps = args.diffusion_steps or max(1, args.max_new_tokens // 4)
        toks = diffusion_generate(model, ids, args.max_new_tokens, steps, block=args.diffusion_block or None, trace=tr)
        return {"mode": "diffusion", "tokens": toks, "text": tk.decode(toks), "passes": tr.passes}
    if args.image:
        from .serve.image import decode_png
        first = model.prefill_multimodal(ids, [decode_png(Path(f).read_bytes()) for f in args.image])
        toks = [first] + [model.decode() for _ in range(args.max_new_tokens - 1)]
        return {"mode": "multimodal", "tokens": toks, "text": tk.decode(toks), "images": len(args.image)}
    depth = resolve_mtp_depth(args.mtp, model.spec.mtp_layers > 0, model.spec.arch)
    mode = "plain"
    extra = {}
    if args.draft_model:
        # a small model drafts, the target verifies: a chain of k tokens, or a token tree under ancestor masks
        from .api import Model
        st = settings_from(args)
        st.graph = bool(args.spec_graph)         # --spec-graph false: the draft model decodes eagerly
        draft = Model.load(args.draft_model, st, device=str(model.engine.device), seed=args.seed + 1)
        if args.spec_budget == "chain":
            from .spec.chain import ChainSpeculator
            sp = ChainSpeculator(model, draft, k=4)
            mode = "draft-chain"
        else:
            from .spec.tree_spec import TreeSpeculator
            sp = TreeSpeculator(model, draft, budget=args.spec_budget, builder=args.tree_builder)
            mode = f"draft-{args.spec_budget}"
        out = sp.generate(ids, args.max_new_tokens, ignore_eos=True)
        extra = {"draft_model": args.draft_model, "spec_budget": args.spec_budget, "tree_builder": args.tree_builder,
                 "rounds": sp.stats.rounds, "acceptance_rate": sp.stats.acceptance_rate,
                 "tokens_per_round": sp.stats.tokens_per_round}
    elif depth > 0:
        from .spec.mtp import generate_mtp
        out = generate_mtp(model, ids, args.max_new_tokens, depth=depth, ignore_eos=args.ignore_eos)
        mode = "mtp"
        extra = {"mtp_depth": depth, "mtp_verify": out.extra.get("verify", "batched"),
                 "accepted_per_round": out.extra.get("accepted_per_round")}
    else:
        out = generate_plain(model, ids, args.max_new_tokens, ignore_eos=args.ignore_eos, graph=args.graph)
        store = model.prefix_store()
        if store is not None:
            extra = {"prefix_cache": {"hits": store.hits, "stored": store.stored, "dir": str(store.root)}}
    if model.engine.kv.compact is not None:
        c = model.engine.kv.compact
        extra = dict(extra, kv={"format": "affine8", "recent": c.recent, **c.stats})
    if trace is not None:
        trace.save(args.dump)
    return {"input_ids": ids, "generated_ids": out.ids, "text": tk.decode(out.ids), "load_ms": model.load_ms,
            "prefill_ms": out.prefill_ms, "capture_ms": out.capture_ms, "decode_ms": out.decode_ms,
            "decode_steps": out.decode_steps, "decode_tok_s": out.decode_tok_s, "graph": bool(args.graph),
            "dump": args.dump, "trace_layer": args.trace_layer, "mode": mode, **extra}


def cmd_bench(args) -> dict:
    """Decode benchmark with the reference's protocol (src/bench.rs:47-51, 89-93, 137-226): at least
    200 timed steps per run after the warm-up, CUDA-event timing per step, median / p10 / p90,
    roofline % = (decode weight bytes + KV bytes read) / time against ``--dram-gb-s``; prefill
    tokens/s against the FLOP model and ``--gemm-tflops``."""
    import torch
    if args.steps < 200:
        raise SystemExit("bench needs --steps >= 200")
    model = _load(args)
    eng, spec = model.engine, model.spec
    eng.use_graph = args.graph and eng.device.type == "cuda"
    g = torch.Generator().manual_seed(1)
    need = args.prompt_tokens + args.warmup + args.steps + 2
    if need > args.capacity:
        raise SystemExit(f"bench needs --capacity >= {need}")
    runs = []
    prefill_tok_s = []
    cuda = eng.device.type == "cuda"
    for _ in range(args.runs):
        eng.reset()
        prompts = [torch.randint(0, spec.vocab, (args.prompt_tokens,), generator=g).tolist() for _ in range(args.batch)]
        seqs = [eng.add_sequence(p) for p in prompts]
        t0 = time.perf_counter()
        eng.prefill(seqs)
        if cuda:
            torch.cuda.synchronize()
        prefill_tok_s.append(args.batch * args.prompt_tokens / (time.perf_counter() - t0))
        for _ in range(args.warmup):
            eng.decode(seqs)
        ms = []
        for _ in range(args.steps):
            if cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(); eng.decode(seqs); e1.record(); torch.cuda.synchronize()
                ms.append(e0.elapsed_time(e1))
            else:
                t = time.perf_counter(); eng.decode(seqs); ms.append((time.perf_counter() - t) * 1e3)
        ms.sort()
        runs.append({"median_ms": statistics.median(ms), "p10_ms": ms[len(ms) // 10], "p90_ms": ms[len(ms) * 9 // 10]})
        for s in seqs:
            eng.free_sequence(s.seq_id)
    med = statistics.median(r["median_ms"] for r in runs)
    ctx = args.prompt_tokens + args.warmup + args.steps // 2
    kv_bytes = args.batch * ctx * spec.layers * 2 * spec.kv_heads * spec.head_dim * 2
    moved = spec.decode_weight_bytes() + kv_bytes
    t_, L, h, f = args.prompt_tokens, spec.layers, spec.hidden, spec.ffn
    flops = 2 * t_ * L * (h * spec.qkv_dim + h * h + 3 * h * f) + 2 * h * spec.vocab + 2 * h * t_ * (t_ + 1) * L
    ptok = statistics.median(prefill_tok_s)
    return {"model": model.name, "batch": args.batch, "steps": args.steps, "warmup": args.warmup, "runs": runs,
            "median_ms": med, "decode_tok_s": args.batch * 1000.0 / med, "graph": eng.use_graph,
            "decode_bytes": moved, "roofline_pct": 100.0 * (moved / (med / 1e3) / 1e9) / args.dram_gb_s,
            "prefill_tok_s": ptok,
            "prefill_roofline_pct": 100.0 * (flops * args.batch * ptok / (args.batch * t_) / 1e12) / args.gemm_tflops}


def cmd_profile(args) -> dict:
    """One decode step or one prefill bracketed by cudaProfilerStart/Stop and an NVTX range
    (src/bench.rs:229-267, src/backend/cuda/profile.rs:5-45)."""
    import torch
    model = _load(args)
    eng = model.engine
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, model.spec.vocab, (args.prompt_tokens,), generator=g).tolist()
    cuda = eng.device.type == "cuda"
    if args.phase == "decode":
        model.prefill(ids)
        model.decode()
    if cuda:
        torch.cuda.synchronize(); torch.cuda.profiler.start(); torch.cuda.nvtx.range_push(f"ff.{args.phase}")
    t0 = time.perf_counter()
    if args.phase == "decode":
        model.decode()
    else:
        model.prefill(ids)
    if cuda:
        torch.cuda.synchronize(); torch.cuda.nvtx.range_pop(); torch.cuda.profiler.stop()
    return {"phase": args.phase, "ms": (time.perf_counter() - t0) * 1e3}


def cmd_inspect(args) -> dict:
    if args.shapes:
        return {"shapes": {k: f().to_json() for k, f in NAMED_SHAPES.items()}}
    from .config import named_shape, read_model_spec
    p = Path(args.model or "")
    if p.is_file() and p.suffix == ".nemo":
        # NeMo archive of a streaming RNN-T: the spec its YAML maps to and the tensor table of the pickled weights
        from dataclasses import asdict
        import torch
        from .loaders.pth import read_nemo
        from .speech.nemo import spec_from_yaml
        text, weights = read_nemo(p)
        try:
            nbytes = sum(r.storage.numel * torch.empty(0, dtype=r.dtype).element_size() for r in weights.records.values())
            if "spk_kernel_type" in text:
                # speaker-attributed recognition: the same encoder / transducer plus the speaker kernels
                from .speech.multitalker import KERNEL_TENSORS, MultitalkerSpec
                mt = MultitalkerSpec.from_yaml(text)
                return {"family": "speech", "architecture": "nemo_multitalker_rnnt", "speakers": mt.speakers, "spec": asdict(mt.asr),
                        "speaker_kernels": [k for k in KERNEL_TENSORS if k + ".weight" in weights.records],
                        "tensors": len(weights.records), "bytes": nbytes}
            return {"family": "speech", "architecture": "nemo_rnnt", "spec": asdict(spec_from_yaml(text)),
                    "tensors": len(weights.records), "bytes": nbytes}
        finally:
            weights.close()
    if p.is_dir():
        from .loaders.checkpoint import inspect_checkpoint
        arch = json.loads((p / "config.json").read_text()).get("architectures", [None])[0] if (p / "config.json").exists() else None
        if arch in ("ParakeetForTDT", "ParakeetForCTC", "CanaryForConditionalGeneration", "Nemotron3_5AsrForRNNT"):
            # speech checkpoints: their own spec classes, contract check included
            from dataclasses import asdict
            from .speech import CanarySpec, ParakeetCtcSpec, ParakeetSpec
            sp = {"ParakeetForTDT": ParakeetSpec, "Nemotron3_5AsrForRNNT": ParakeetSpec, "ParakeetForCTC": ParakeetCtcSpec,
                  "CanaryForConditionalGeneration": CanarySpec}[arch].read(p)
            info = inspect_checkpoint(p)
            return {"family": "speech", "architecture": arch, "spec": asdict(sp), "expected_tensors": len(sp.expected_tensors()), **info}
        if arch == "Nemotron3DiarizationForAudioFrameClassification":
            from dataclasses import asdict
            from .speech.diarization import DiarizationSpec
            sp = DiarizationSpec.from_json(json.loads((p / "config.json").read_text()), json.loads((p / "processor_config.json").read_text()))
            return {"family": "speech", "architecture": arch, "spec": asdict(sp), "expected_tensors": len(sp.expected_tensors()),
                    "max_encoder_rows": sp.max_encoder_rows(), **inspect_checkpoint(p)}
        spec = read_model_spec(p)
        return {"spec": spec.to_json(), **inspect_checkpoint(p)}
    return {"spec": named_shape(args.model).to_json()}


def cmd_tokenize(args) -> dict:
    from .loaders.tokenizer import ByteTokenizer, load_tokenizer
    tk = (load_tokenizer(args.model) if args.model and Path(args.model).is_dir() else None) or ByteTokenizer()
    ids = tk.encode(args.prompt)
    return {"ids": ids, "count": len(ids)}


def cmd_calibrate(args) -> dict:
    from .planner.calibrate import calibrate
    return calibrate(args.model, settings_from(args), force=args.force, cpu=args.cpu)


def cmd_embed(args) -> dict:
    from .loaders.tokenizer import ByteTokenizer
    model = _load(args)
    tk = model.tokenizer or ByteTokenizer(model.spec.vocab)
    if model.spec.extra.get("bidirectional"):
        # embedding encoders: bidirectional attention, mean pooling, dense head, L2 normalisation
        from .models.encoder import embed_texts
        vec = [float(v) for v in embed_texts(model, [tk.encode(args.prompt)])[0].cpu().tolist()]
    else:
        from .models.embedding import embed_text
        vec = embed_text(model, tk.encode(args.prompt))
    return {"dim": len(vec), "embedding": vec}


def cmd_transcribe(args) -> None:
    """Speech recognition of one audio file (src/main.rs:861-990 of the reference: same formats, output file guard)."""
    from .speech import load_audio, load_model
    if not args.model:
        raise SystemExit("transcribe needs --model")
    if str(args.model).endswith(".nemo"):
        # NeMo archive of a streaming RNN-T (end-of-utterance models): --stream cuts the text into timed utterances
        from .loaders.pth import read_nemo_member
        from .speech.nemo import transcribe_nemo
        out_path = check_output_path(args.output, None) if args.output else None
        wave = load_audio(args.input, 16000)
        if b"spk_kernel_type" in read_nemo_member(args.model, "model_config.yaml"):
            # speaker-attributed recognition: one transcript per speaker the diarizer hears
            from .speech.multitalker import transcribe_multitalker
            if not args.diarization_model:
                raise SystemExit("a multitalker archive needs --diarization-model (speaker activity selects its lanes)")
            if args.format not in ("txt", "json"):
                raise SystemExit("speaker-attributed transcripts come as txt or json")
            res = transcribe_multitalker(args.model, args.diarization_model, wave, "cpu" if args.cpu else f"cuda:{args.device}",
                                         stream_diarizer=args.stream, masked=args.masked_asr)
            text = res.to_text() if args.format == "txt" else res.to_json() + "\n"
            (out_path.write_text(text) if out_path is not None else sys.stdout.write(text))
            return
        if args.diarization_model or args.masked_asr:
            raise SystemExit("--diarization-model / --masked-asr apply to multitalker archives")
        result = transcribe_nemo(args.model, wave, "cpu" if args.cpu else f"cuda:{args.device}", stream=args.stream)
        text = {"txt": result.text + "\n", "json": result.to_json() + "\n", "srt": result.to_srt(), "vtt": result.to_vtt()}[args.format]
        (out_path.write_text(text) if out_path is not None else sys.stdout.write(text))
        return
    arch = json.loads((Path(args.model) / "config.json").read_text()).get("architectures", [None])[0]
    if arch not in ("ParakeetForTDT", "ParakeetForCTC", "CanaryForConditionalGeneration", "Nemotron3_5AsrForRNNT"):
        raise SystemExit(f"unsupported transcription architecture {arch}")
    out_path = check_output_path(args.output, args.model) if args.output else None
    device = "cpu" if args.cpu else f"cuda:{args.device}"
    model = load_model(args.model, device)
    wave = load_audio(args.input, model.spec.mel.sampling_rate)
    if arch == "Nemotron3_5AsrForRNNT":
        # the prompt id conditions the encoder rows on a language: --source-lang names an entry of the prompt dictionary
        table = dict(model.spec.prompt_dictionary)
        if args.source_lang in table:
            model.decoder.prompt_id = table[args.source_lang]
        elif args.source_lang != "en":
            raise SystemExit(f"--source-lang {args.source_lang} is not in the prompt dictionary ({', '.join(sorted(table))})")
        args.source_lang = "en"
    if args.stream:
        # cache-aware streaming encoders only: audio goes in 320 ms pieces, one JSON line per piece that produced tokens
        from .speech import ParakeetModel, StreamingRecognizer
        enc = getattr(model.spec, "encoder", None)
        if not isinstance(model, ParakeetModel) or enc is None or enc.chunk_size <= 0 or model.spec.mel.normalize:
            raise SystemExit(f"streaming transcription is not available for this {arch} checkpoint (no chunk-wise encoder context)")
        rec = StreamingRecognizer(model)
        piece = model.spec.mel.sampling_rate * 32 // 100
        for at in range(0, wave.numel(), piece):
            nxt = min(wave.numel(), at + piece)
            new = rec.push(wave[at:nxt], last=nxt == wave.numel())
            if new and model.tokenizer is not None:
                sys.stderr.write(json.dumps({"seconds": nxt / model.spec.mel.sampling_rate, "tokens": new,
                                             "text": model.tokenizer.decode(new)}) + "\n")
        result = rec.transcription()
        text = {"txt": result.text + "\n", "json": result.to_json() + "\n", "srt": result.to_srt(), "vtt": result.to_vtt()}[args.format]
        (out_path.write_text(text) if out_path is not None else sys.stdout.write(text))
        return
    if arch == "CanaryForConditionalGeneration":
        result = model.transcribe([wave], args.source_lang, args.target_lang, not args.no_pnc)[0]
    else:
        if (args.source_lang, args.target_lang, args.no_pnc) != ("en", "en", False):
            raise SystemExit(f"--source-lang / --target-lang / --no-pnc apply to Canary models, not to {arch}")
        result = model.transcribe([wave])[0]
    text = {"txt": result.text + "\n", "json": result.to_json() + "\n", "srt": result.to_srt(), "vtt": result.to_vtt()}[args.format]
    if out_path is not None:
        out_path.write_text(text)
    else:
        sys.stdout.write(text)


def cmd_diarize(args) -> None:
    """Who spoke when, for one audio file (src/main.rs `diarize` of the reference: RTTM or JSON segments)."""
    from .speech import load_audio
    from .speech.diarization import ARCHITECTURE, load_model
    from .speech.transcript import to_rttm
    if not args.model:
        raise SystemExit("diarize needs --model")
    arch = json.loads((Path(args.model) / "config.json").read_text()).get("architectures", [None])[0]
    if arch != ARCHITECTURE:
        raise SystemExit(f"unsupported diarization architecture {arch}")
    if not (0.0 <= args.threshold <= 1.0):
        raise SystemExit("--threshold must lie in [0, 1]")
    out_path = check_output_path(args.output, args.model) if args.output else None
    model = load_model(args.model, "cpu" if args.cpu else f"cuda:{args.device}")
    if args.mode is not None and not args.stream:
        raise SystemExit("--mode applies to --stream")
    wave = load_audio(args.input, model.spec.mel.sampling_rate)
    segments = model.diarize(wave, stream=args.stream, threshold=args.threshold, mode=args.mode)
    if args.format == "rttm":
        stem = "".join(c if not c.isspace() else "_" for c in Path(args.input).stem) or "audio"
        text = to_rttm(stem, segments)
    else:
        text = json.dumps([{"start": s.start, "end": s.end, "speaker": s.text} for s in segments]) + "\n"
    if out_path is not None:
        out_path.write_text(text)
    else:
        sys.stdout.write(text)


def cmd_to_3d(args) -> dict:
    """The decode tail of image-to-3D: the shape decoder's sparse output -> surface -> post-processing -> mesh file
    (src/main.rs `to-3d` of the reference ends the same way; the generator in front of it is not part of this build,
    so the command starts from the decoder's saved output)."""
    import torch
    from .loaders.safetensors_io import SafetensorsFile
    from .ops import mesh_ops
    from .utils import media, mesh_post
    if args.model:
        raise SystemExit("to-3d starts from saved decoder output (the image-to-3D generator is not built): pass no --model")
    out = check_output_path(args.output, None)
    if out.suffix not in (".ply", ".obj"):
        raise SystemExit("--output must end in .ply or .obj")
    sf = SafetensorsFile(args.input)
    try:
        t = {n: sf.tensor(n).clone() for n in sf.tensors}
    finally:
        sf.close()
    dev = "cpu" if args.cpu else f"cuda:{args.device}"
    if "coords" not in t:
        raise SystemExit("the input holds no `coords` tensor")
    coords = t["coords"].to(torch.int32).to(dev)
    if "fields" in t:
        if args.resolution <= 0:
            raise SystemExit("dual-grid fields need --resolution")
        v, f = mesh_ops.dual_grid_mesh(coords, t["fields"].float().to(dev), args.resolution)
        kind = "dual_grid"
    elif all(k in t for k in ("cubes", "positions", "scalar")):
        v, f = mesh_ops.dual_contour_mesh(coords, t["cubes"].to(dev), t["positions"].float().to(dev), t["scalar"].float().to(dev))
        kind = "dual_contour"
    elif "scalar" in t:
        # values on the shared corner lattice of the cubes, in the lexicographic corner order
        from .ops import sparse_sites
        corners, cubes, _, _ = sparse_sites.cube_corners(coords)
        if t["scalar"].numel() != corners.shape[0]:
            raise SystemExit(f"`scalar` has {t['scalar'].numel()} values for {corners.shape[0]} cube corners")
        v, f = mesh_ops.dual_contour_mesh(coords, cubes, corners[:, 1:].float(), t["scalar"].float().reshape(-1).to(dev))
        kind = "dual_contour"
    else:
        raise SystemExit("the input holds neither `fields` nor `scalar` (with or without `cubes` / `positions`)")
    v, f, report = mesh_post.finish_mesh(v, f, args.min_component, args.fill_holes, args.faces, args.unit_ball)
    with open(out, "wb") as fh:
        (media.write_ply if out.suffix == ".ply" else media.write_obj)(fh, media.Mesh(v, f))
    return {"surface": kind, "output": str(out), **report}


def cmd_serve(args) -> None:
    from .loaders.tokenizer import read_chat_template
    from .serve.http import run
    model = _load(args)
    depth = resolve_mtp_depth(args.mtp, model.spec.mtp_layers > 0, model.spec.arch) if args.mtp is not None else 0
    if depth > 0 and args.tp > 1:
        raise SystemExit("serve --mtp with --tp is not supported")
    tmpl = read_chat_template(args.model) if Path(args.model).is_dir() else None
    engine = None
    if args.tp > 1:
        # rank 0 serves; the other ranks execute the engine calls it announces
        import torch.distributed as dist
        from .parallel.driver import EngineLeader, follow
        host_group = dist.new_group(backend="gloo")
        if _world()[1] != 0:
            follow(model.engine, host_group)
            return
        engine = EngineLeader(model.engine, host_group)
    try:
        run(model, port=args.port, allow_sampling=args.allow_sampling, chat_template=tmpl, mtp_depth=depth, engine=engine)
    finally:
        if engine is not None:
            engine.stop()


def cmd_verify(args) -> dict:
    from .utils.verify import compare_traces
    return compare_traces(args.trace, args.reference, getattr(args, "limits", None))


def cmd_compare_log(args) -> dict:
    from .utils.verify import compare_logs
    return compare_logs(args.a, args.b)


def cmd_spec(args) -> dict:
    from .spec.drivers import run_spec_tool
    model = _load(args)
    return run_spec_tool(args.command, model, args.prompt_tokens, args.max_new_tokens, args.mtp, args.strict)


def cmd_dspark(args) -> dict:
    from .api import Model
    from .spec.drivers import run_dspark_tool
    if getattr(args, "trace", None) and not Path(args.trace).exists():
        check_output_path(args.trace, args.model)
    model = _load(args)
    st = settings_from(args)
    st.graph = bool(args.spec_graph)
    draft = Model.load(args.draft_model, st, device=str(model.engine.device), seed=args.seed + 1)
    budget = args.spec_budget if args.spec_budget != "chain" else "tree16"
    return run_dspark_tool(args.command, model, draft, args.prompt_tokens, args.max_new_tokens, budget=budget,
                           builder=args.tree_builder, trace_path=getattr(args, "trace", None), strict=args.strict)


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    args = _global_parser().parse_args(argv)
    check_flags(args)
    rc = relaunch_tp(args, argv)
    if rc is not None:
        return rc
    handlers = {"generate": cmd_generate, "bench": cmd_bench, "profile": cmd_profile, "inspect": cmd_inspect,
                "tokenize": cmd_tokenize, "calibrate": cmd_calibrate, "embed": cmd_embed, "verify": cmd_verify,
                "compare-prefill": cmd_verify, "compare-log": cmd_compare_log, "verify-spec": cmd_spec,
                "bench-spec": cmd_spec, "profile-spec": cmd_spec, "to-3d": cmd_to_3d, **{t: cmd_dspark for t in DSPARK_TOOLS}}
    if args.command == "serve":
        cmd_serve(args)
        return 0
    if args.command == "transcribe":
        cmd_transcribe(args)
        return 0
    if args.command == "diarize":
        cmd_diarize(args)
        return 0
    out = handlers[args.command](args)
    if _world()[1] == 0:
        print(json.dumps(out, default=str))
    return 0


if __name__ == "__main__":
    sys.exit(main())
