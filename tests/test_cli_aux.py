"""CLI parsing and JSON output, output-path guard, trace / verify tools, prefix cache, the
calibration closure and cache -- all on CPU with the tiny decoder."""
import json

import pytest
import torch

from flyingfish_b200 import cli
from flyingfish_b200.api import Model, generate_plain
from flyingfish_b200.config import Settings
from flyingfish_b200.planner.calibrate import (Closure, ClosureError, ClosureState, calibrate, check_runtime_dir,
                                               host_memory_limit)


def _run(argv, capsys):
    assert cli.main(argv) == 0
    return json.loads(capsys.readouterr().out.strip().splitlines()[-1])


def test_generate_json_fields(capsys):
    out = _run(["--model", "tiny-llama", "--cpu", "--capacity", "128", "generate", "--tokens", "1,2,3,4", "--max-new-tokens", "5",
                "--ignore-eos"], capsys)
    for k in ("input_ids", "generated_ids", "text", "load_ms", "prefill_ms", "capture_ms", "decode_ms", "decode_steps",
              "decode_tok_s", "graph", "dump", "trace_layer", "mode"):
        assert k in out
    assert out["input_ids"] == [1, 2, 3, 4] and len(out["generated_ids"]) == 5 and out["mode"] == "plain"
    assert out["decode_steps"] == 4      # the first id comes from prefill


def test_global_options_come_first_and_model_is_required(capsys, monkeypatch):
    monkeypatch.delenv("FLYINGFISH_MODEL", raising=False)
    with pytest.raises(SystemExit):
        cli.main(["generate", "--tokens", "1"])
    with pytest.raises(SystemExit):
        cli.main(["--model", "tiny-llama", "--cpu", "generate", "--tokens", "1", "--prompt", "x"])
    with pytest.raises(SystemExit):
        cli.main(["--model", "tiny-llama", "--cpu", "--capacity", "8", "generate", "--tokens", "1,2,3", "--max-new-tokens", "9"])
    monkeypatch.setenv("FLYINGFISH_MODEL", "tiny-llama")
    out = _run(["--cpu", "--capacity", "64", "generate", "--prompt", "hi", "--max-new-tokens", "2", "--ignore-eos"], capsys)
    assert out["input_ids"] == [104, 105]


def test_tokens_file_forms(tmp_path):
    class A: pass
    for content, want in (([1, 2], [1, 2]), ({"input_ids": [3, 4]}, [3, 4]), ([[5, 6], [7]], [5, 6])):
        p = tmp_path / f"t{len(str(content))}.json"
        p.write_text(json.dumps(content))
        a = A(); a.tokens = None; a.tokens_file = str(p)
        assert cli.parse_tokens_arg(a) == want


def test_output_path_guard(tmp_path):
    (tmp_path / "exists.bin").write_text("x")
    with pytest.raises(SystemExit):
        cli.check_output_path(tmp_path / "exists.bin", None)
    (tmp_path / "models").mkdir()
    with pytest.raises(SystemExit):
        cli.check_output_path(tmp_path / "models" / "new.bin", None)
    md = tmp_path / "ckpt"; md.mkdir()
    with pytest.raises(SystemExit):
        cli.check_output_path(md / "trace.safetensors", str(md))
    assert cli.check_output_path(tmp_path / "fine.bin", str(md)).name == "fine.bin"


def test_mtp_depth_resolution():
    assert cli.resolve_mtp_depth(None, False, "llama") == 0
    assert cli.resolve_mtp_depth(None, True, "llama") == 4
    assert cli.resolve_mtp_depth(None, True, "deepseek_v3") == 0
    assert cli.resolve_mtp_depth(2, True, "deepseek_v3") == 2
    with pytest.raises(SystemExit):
        cli.resolve_mtp_depth(2, False, "llama")


def test_inspect_tokenize_and_bench_floor(capsys):
    out = _run(["inspect", "--shapes"], capsys)
    assert "llama3-8b-shape" in out["shapes"] and out["shapes"]["deepseek-v3-shape"]["mla"]["kv_lora_rank"] == 512
    out = _run(["tokenize", "--prompt", "abc"], capsys)
    assert out == {"ids": [97, 98, 99], "count": 3}
    with pytest.raises(SystemExit):
        cli.main(["--model", "tiny-llama", "--cpu", "bench", "--steps", "10"])


def test_dump_and_verify_roundtrip(tmp_path, capsys):
    a, b = tmp_path / "a.safetensors", tmp_path / "b.safetensors"
    base = ["--model", "tiny-llama", "--cpu", "--capacity", "64", "generate", "--tokens", "5,6,7", "--max-new-tokens", "2", "--ignore-eos"]
    _run(base + ["--dump", str(a)], capsys)
    _run(base + ["--dump", str(b), "--trace-layer", "1"], capsys)
    with pytest.raises(SystemExit):
        cli.main(base + ["--dump", str(tmp_path / "c.st"), "--graph"])
    from flyingfish_b200.utils.verify import compare_traces, tensor_metrics
    rep = compare_traces(a, a)
    assert rep["ok"] and all(m["max_abs"] == 0 for m in rep["tensors"].values())
    assert any(k.endswith("logits") and "top_two_margin" in m for k, m in rep["tensors"].items())
    rep = compare_traces(b, a)
    assert not rep["ok"] and any("missing_in" in m for m in rep["tensors"].values())
    m = tensor_metrics(torch.tensor([1.0, 2.0]), torch.tensor([1.0, 2.0078125]))
    assert m["bf16_bit_mismatches"] == 0 or m["half_ulp_ratio"] >= 1.0
    lim = tmp_path / "lim.json"; lim.write_text(json.dumps({"*": 1e-9}))
    assert compare_traces(a, a, lim)["ok"]


def test_compare_logs(tmp_path):
    from flyingfish_b200.utils.verify import compare_logs
    (tmp_path / "a.log").write_text('{"generated_ids": [1, 2]}\n')
    (tmp_path / "b.log").write_text('noise\n{"generated_ids": [1, 3]}\n')
    assert not compare_logs(tmp_path / "a.log", tmp_path / "b.log")["ok"]
    assert compare_logs(tmp_path / "a.log", tmp_path / "a.log")["ok"]


def test_prefix_cache_roundtrip(tmp_path):
    from flyingfish_b200.utils.prefix_cache import PrefixError, restore_prefix, save_prefix
    m = Model.load("tiny-llama", Settings(capacity=256, max_batch=2, graph=False), device="cpu", seed=0)
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, 2048, (70,), generator=g).tolist()
    want = generate_plain(m, ids, 6, ignore_eos=True, graph=False).ids
    m.reset()
    seq = m.engine.add_sequence(ids[:66])
    m.engine.prefill([seq])
    pkg = save_prefix(m, seq, tmp_path / "pfx")
    m.reset()
    seq2 = restore_prefix(m, pkg)
    assert m.engine.kv.seqs[seq2.seq_id].length == 66
    seq2.prompt = ids                      # continue with the rest of the prompt
    first = m.engine.prefill([seq2])[0]
    got = [first] + [m.engine.decode([seq2])[0] for _ in range(5)]
    assert got == want
    with pytest.raises(PrefixError):
        save_prefix(m, seq2, pkg)          # no overwrite
    other = Model.load("tiny-llama", Settings(capacity=256, max_batch=2, graph=False, kv_format="affine8"), device="cpu")
    with pytest.raises(PrefixError, match="different"):
        restore_prefix(other, pkg)
    man = json.loads((pkg / "manifest.json").read_text()); man["tokens"][0] ^= 1
    (pkg / "manifest.json").write_text(json.dumps(man))
    m.reset()
    with pytest.raises(PrefixError, match="corrupt"):
        restore_prefix(m, pkg)


def test_closure_state_machine_and_calibration_cache(tmp_path):
    c = Closure()
    c.measure("x"); c.declare_shape((1, 2, 3))
    with pytest.raises(ClosureError):
        c.capture()
    c.freeze()
    with pytest.raises(ClosureError):
        c.measure("late")
    c.capture(); c.declare_shape((4, 5, 6)); c.ready()
    assert c.state is ClosureState.READY and c.captures == 1
    with pytest.raises(ClosureError):
        c.declare_shape((7, 8, 9))
    c.declare_shape((1, 2, 3))
    with pytest.raises(ClosureError):
        check_runtime_dir(tmp_path / "models" / "rt")
    assert host_memory_limit() > 0
    st = Settings(runtime_dir=str(tmp_path / "rt"))
    d1 = calibrate("qwen3-moe-tiny", st, cpu=True)
    assert not d1["cached"] and d1["disk_bytes_s"] > 0 and "cpu_service" in d1
    assert calibrate("qwen3-moe-tiny", st, cpu=True)["cached"]
    assert not calibrate("qwen3-moe-tiny", st, force=True, cpu=True)["cached"]


def test_generate_for_the_other_model_families(tmp_path, capsys):
    """Diffusion canvas, embedding encoder, image input, hybrid and Gemma layouts through the command line."""
    import sys as _sys
    from pathlib import Path
    _sys.path.insert(0, str(Path(__file__).parent))
    from test_vision import _png
    base = ["--cpu", "--capacity", "256"]

    def run(*argv):
        return _run(list(argv), capsys)

    d = run(*base, "--model", "tiny-diffusion", "generate", "--tokens", "5,6,7", "--max-new-tokens", "8",
            "--diffusion-steps", "2")
    assert d["mode"] == "diffusion" and len(d["tokens"]) == 8 and d["passes"] == 2 and 2046 not in d["tokens"]
    e = run(*base, "--model", "tiny-embed", "embed", "--prompt", "hello")
    assert e["dim"] == 256 and abs(sum(v * v for v in e["embedding"]) - 1.0) < 1e-3
    img = tmp_path / "a.png"
    img.write_bytes(_png(64, 64, 9))
    v = run(*base, "--model", "tiny-vl", "generate", "--tokens", "5,2047,7", "--image", str(img), "--max-new-tokens", "3")
    assert v["mode"] == "multimodal" and len(v["tokens"]) == 3 and v["images"] == 1
    for name in ("tiny-hybrid", "tiny-gemma"):
        g = run(*base, "--model", name, "generate", "--tokens", "5,6,7,8", "--max-new-tokens", "4", "--ignore-eos")
        assert len(g["generated_ids"]) == 4


# ---- every flag changes behaviour or is refused ---------------------------------------------------------------------
BASE = ["--model", "tiny-llama", "--cpu", "--capacity", "256"]
GEN = ["generate", "--tokens", "5,6,7,8,9,10,11", "--max-new-tokens", "9", "--ignore-eos"]


def test_flags_without_an_implementation_are_refused(capsys):
    for extra in (["--kv-format", "affine8", "--draft-model", "tiny-llama"], ["--kv-format", "affine8", "--prefix-cache", "true"],
                  ["--tp", "2"], ["--spec-budget", "tree16"], ["--spec-graph", "false"]):
        with pytest.raises(SystemExit):
            cli.main(BASE + extra + GEN)
    with pytest.raises(SystemExit):      # a draft model only makes sense for generate
        cli.main(BASE + ["--draft-model", "tiny-llama", "tokenize", "--prompt", "x"])
    with pytest.raises(SystemExit):      # the server's scheduler does not consult the prefix store
        cli.main(BASE + ["--prefix-cache", "true", "serve"])


def test_kv_format_affine8_seals_old_groups_and_keeps_decoding(capsys):
    """``--kv-format affine8 --kv-recent 128``: groups older than the recent window move to the 8-bit store (their BF16
    blocks are released) and decoding goes on over sink + sealed groups + recent pages."""
    g = torch.Generator().manual_seed(21)
    long = ["generate", "--tokens", ",".join(map(str, torch.randint(0, 2048, (300,), generator=g).tolist())),
            "--max-new-tokens", "40", "--ignore-eos"]
    base = ["--model", "tiny-llama", "--cpu", "--capacity", "1024"]
    plain = _run(base + long, capsys)
    packed = _run(base + ["--kv-format", "affine8", "--kv-recent", "128"] + long, capsys)
    assert len(packed["generated_ids"]) == 40 and "kv" not in plain
    # 300 + 40 tokens with 128 recent: positions below 128 are sealed (1 group, block 1 released; block 0 is the sink)
    assert packed["kv"]["format"] == "affine8" and packed["kv"]["sealed_groups"] == 1 and packed["kv"]["released_blocks"] == 1
    # 8-bit keys and values perturb the logits slightly: the continuations agree at the start
    agree = next((i for i, (a, b) in enumerate(zip(plain["generated_ids"], packed["generated_ids"])) if a != b), 40)
    assert agree >= 3, (plain["generated_ids"], packed["generated_ids"])


def test_draft_model_flags_select_the_speculator(capsys):
    plain = _run(BASE + GEN, capsys)
    chain = _run(BASE + ["--draft-model", "tiny-llama"] + GEN, capsys)
    assert chain["mode"] == "draft-chain" and chain["rounds"] > 0
    assert chain["generated_ids"] == plain["generated_ids"]         # speculation never changes greedy output
    for builder in ("waves", "serial", "markov"):
        tree = _run(BASE + ["--draft-model", "tiny-llama", "--spec-budget", "tree16", "--tree-builder", builder] + GEN, capsys)
        assert tree["mode"] == "draft-tree16" and tree["tree_builder"] == builder
        assert tree["generated_ids"] == plain["generated_ids"]


def test_prefix_cache_flag_restores_a_stored_prompt(capsys, tmp_path):
    args = BASE + ["--prefix-cache", "true", "--runtime-dir", str(tmp_path)]
    plain = _run(BASE + GEN, capsys)
    first = _run(args + GEN, capsys)
    assert first["prefix_cache"] == {"hits": 0, "stored": 1, "dir": str(tmp_path / "prefix")}
    second = _run(args + GEN, capsys)
    assert second["prefix_cache"]["hits"] == 1 and second["prefix_cache"]["stored"] == 0
    assert first["generated_ids"] == second["generated_ids"] == plain["generated_ids"]
    # a longer prompt that starts with the stored one restores it and computes only the rest
    longer = ["generate", "--tokens", "5,6,7,8,9,10,11,12,13", "--max-new-tokens", "4", "--ignore-eos"]
    a = _run(BASE + longer, capsys)
    b = _run(args + longer, capsys)
    assert b["prefix_cache"]["hits"] == 1 and a["generated_ids"] == b["generated_ids"]


def test_mtp_backend_serves_one_request_at_a_time():
    """``serve --mtp``: requests are generated by MTP speculation (same tokens as plain greedy decoding), one at a
    time; a second request while one runs is refused as busy."""
    import asyncio
    from flyingfish_b200.serve.backend import Busy, MtpBackend
    model = Model.load("tiny-llama", Settings(capacity=256, max_batch=2, graph=False), device="cpu", seed=0)
    ids = list(range(7, 27))
    plain = generate_plain(model, ids, 10, ignore_eos=True, graph=False).ids
    model.reset()

    async def main():
        be = MtpBackend(model, depth=2)
        be.start()
        try:
            req, q = be.add_request(ids, 10, ignore_eos=True)
            with pytest.raises(Busy):
                be.add_request(ids, 4, ignore_eos=True)
            toks = []
            while True:
                ev = await asyncio.wait_for(q.get(), timeout=60)
                if ev.kind == "tokens":
                    toks += ev.tokens
                else:
                    assert ev.kind == "done" and ev.finish_reason == "length"
                    break
            assert toks == plain
            assert be.spec.stats.rounds > 0
        finally:
            be.shutdown()
    asyncio.run(main())


def test_engine_leader_and_follower_execute_the_same_calls():
    """Tensor-parallel serving: rank 0 announces every engine call, the follower executes it on its own engine. Two
    gloo ranks, each with its own CPU engine, must end with identical sequences."""
    # process groups are per process, so the two ranks are child processes
    import multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_driver_rank, args=(r, 29631, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=180) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
    by_rank = dict(got)
    assert by_rank[0] == by_rank[1] and len(by_rank[0]) == 2 and all(len(o) == 6 for o in by_rank[0])


def _driver_rank(rank, port, q):
    import os
    import torch.distributed as dist
    from flyingfish_b200.engine.scheduler import Request, Scheduler
    from flyingfish_b200.parallel.driver import EngineLeader, follow
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE="2")
    dist.init_process_group("gloo", rank=rank, world_size=2)
    model = Model.load("tiny-llama", Settings(capacity=128, max_batch=4, graph=False), device="cpu", seed=0)
    eng = model.engine
    if rank == 0:
        lead = EngineLeader(eng, dist.group.WORLD)
        sch = Scheduler(lead)
        reqs = [Request(prompt=list(range(3 + i, 20 + i)), max_tokens=6, ignore_eos=True) for i in range(2)]
        for r in reqs:
            sch.submit(r)
        sch.run_until_idle()
        lead.stop()
        q.put((0, [r.output for r in reqs]))
    else:
        outs = {}
        orig_free = eng.free_sequence

        def free(seq_id):                 # keep what the follower generated before the leader frees the sequence
            if seq_id in eng.seqs:
                outs[seq_id] = list(eng.seqs[seq_id].output)
            orig_free(seq_id)
        eng.free_sequence = free
        follow(eng, dist.group.WORLD)
        q.put((1, [outs[k] for k in sorted(outs)]))
    dist.destroy_process_group()


def test_draft_model_tools(capsys, tmp_path):
    """The draft-model tools: each reports that speculation leaves greedy decoding unchanged; the replay tools write a
    trace on the first run and reproduce it on the second."""
    base = BASE + ["--draft-model", "tiny-llama"]
    small = ["--prompt-tokens", "20", "--max-new-tokens", "10"]
    out = _run(base + ["check-tree-greedy"] + small + ["--strict"], capsys)
    assert out["identical_to_greedy"] and out["budget"] == "tree16" and out["rounds"] > 0
    out = _run(base + ["compare-tree-builders"] + small, capsys)
    assert out["identical_to_greedy"] and set(out["builders"]) == {"waves", "serial", "markov"}
    # the Markov head needs one draft forward per depth and round, the per-node builders one per expanded node
    assert out["builders"]["markov"]["draft_forwards"] < out["builders"]["waves"]["draft_forwards"]
    out = _run(base + ["compare-tree-padding"] + small, capsys)
    assert out["identical_to_greedy"] and [out["budgets"][b]["rows"] for b in ("tree16", "tree32", "tree64")] == [16, 32, 64]
    out = _run(base + ["compare-spec-graph"] + small, capsys)
    assert out["identical"] and out["identical_to_greedy"]
    for tool in ("replay-draft", "replay-tree"):
        trace = tmp_path / f"{tool}.json"
        first = _run(base + [tool] + small + ["--trace", str(trace)], capsys)
        assert first["identical_to_greedy"] and first["trace_written"] == str(trace)
        second = _run(base + [tool] + small + ["--trace", str(trace)], capsys)
        assert second["replay_matches_trace"] is True
    with pytest.raises(SystemExit):
        cli.main(BASE + ["check-tree-greedy"])            # needs a draft model
