"""Expert tiering: capacity / admission arithmetic, the residency state machine, the native CPU
expert FFN and reader pool, and the tiered provider end to end (results independent of where an
expert lives)."""
import os

import pytest
import torch

from flyingfish_b200.experts import native
from flyingfish_b200.experts.plan import (Admission, CpuService, ExpertGeometry, PlanError, Tier, TransferRates,
                                          admission_budget, initial_residency, plan_capacity, seed_scores)
from flyingfish_b200.experts.runtime import Residency, Route
from flyingfish_b200.ops import ref


def test_capacity_split_and_tiers():
    geo = ExpertGeometry(layers=4, experts_per_layer=16, top_k=2, slot_bytes=100)
    cap = plan_capacity(geo, device_expert_bytes=100 * 30, host_bytes=100 * 20, rates=TransferRates(), admission_cap=2)
    assert cap.gpu_slots == 30 and cap.slots_per_layer == [8, 8, 7, 7]      # remainder to the low layers
    assert cap.host_blocks == 20 and cap.disk_experts == 64 - 30 - 20 and cap.spare_blocks == 2
    full = plan_capacity(geo, 100 * 1000, 0, TransferRates())
    assert full.all_resident and full.slots_per_layer == [16] * 4
    half = plan_capacity(geo, 100 * 1000, 100 * 1000, TransferRates(), resident_fraction=0.5)
    assert half.gpu_slots == 32 and half.host_blocks == 32 and half.disk_experts == 0
    with pytest.raises(PlanError):
        plan_capacity(geo, 100 * 5, 0, TransferRates())


def test_admission_budget():
    geo = ExpertGeometry(layers=10, experts_per_layer=8, top_k=2, slot_bytes=10_000_000)
    a = admission_budget(geo, TransferRates(h2d_bytes_s=50e9, d2h_bytes_s=25e9, copy_engines=2), CpuService(per_expert_s=1e-3))
    assert a.bytes_per_token == pytest.approx(10 * 1e-3 * 25e9) and a.hard_cap == 25
    b = admission_budget(geo, TransferRates(h2d_bytes_s=50e9, d2h_bytes_s=50e9, copy_engines=1), CpuService(per_expert_s=1e-3))
    assert b.bytes_per_token == pytest.approx(10 * 1e-3 * 25e9)


def test_initial_residency_and_seeds():
    freq = [[0, 5, 5, 1], [3, 0, 0, 0]]
    assert initial_residency(freq, [2, 2]) == [[1, 2], [0, 1]]
    assert seed_scores([1, 3], top_k=2) == [12 * 1 * 2 / 4, 12 * 3 * 2 / 4]
    assert seed_scores([0, 0], 2) == [0.0, 0.0]


def test_residency_token_loop():
    geo = ExpertGeometry(layers=1, experts_per_layer=6, top_k=2, slot_bytes=10)
    cap = plan_capacity(geo, 10 * 3, 10 * 10, TransferRates())
    res = Residency(geo, cap, Admission(1e9, hard_cap=1))
    moves = res.begin_request([[9, 8, 7, 0, 0, 0]])
    assert sorted(m.expert_in for m in moves) == [0, 1, 2] and res.resident(0) == [0, 1, 2]
    assert res.ledger.count(Tier.GPU) == 3
    gens = [res.generation[0][res.slot_of[0][e]] for e in (0, 1, 2)]
    # expert 4 is routed repeatedly while 2 cools down: it must replace the coldest unrouted resident
    admitted = []
    for _ in range(60):
        res.begin_token()
        d = res.dispatch(0, [Route(0, 0, 0, 0.5), Route(0, 1, 4, 0.5)])
        admitted += res.finish_token()
        if admitted:
            break
    assert [m.expert_in for m in admitted] == [4]
    assert admitted[0].expert_out in (1, 2) and admitted[0].generation == gens[0] + 1
    assert 4 in res.resident(0) and res.ledger.where(0, admitted[0].expert_out) == Tier.HOST
    res.begin_token()
    d = res.dispatch(0, [Route(0, 0, 4, 1.0), Route(0, 1, 5, 1.0)])
    assert [r.expert for r in d.hits] == [4] and [r.expert for r in d.host] == [5]
    with pytest.raises(AssertionError):
        res.begin_token()                     # finish_token missing
    res.finish_token()
    with pytest.raises(ValueError):
        res.begin_token(); res.dispatch(0, [Route(0, 0, 99, 1.0)])


def test_victim_is_never_a_routed_expert_and_cap_holds():
    geo = ExpertGeometry(layers=2, experts_per_layer=4, top_k=2, slot_bytes=10)
    cap = plan_capacity(geo, 10 * 4, 10 * 10, TransferRates())
    res = Residency(geo, cap, Admission(1e9, hard_cap=1))
    res.begin_request([[5, 4, 0, 0], [5, 4, 0, 0]])
    for l in range(2):
        res.score[l][2] = res.score[l][3] = 50.0
    res.begin_token()
    for l in range(2):
        res.dispatch(l, [Route(0, 0, 0, 0.5), Route(0, 1, 1, 0.5), Route(1, 0, 2, 0.5), Route(1, 1, 3, 0.5)])
    assert res.finish_token() == []            # every resident was routed: no victim available
    res.begin_token()
    for l in range(2):
        res.dispatch(l, [Route(0, 0, 2, 1.0)])
    assert len(res.finish_token()) == 1        # hard cap of one admission per token across layers


def test_cpu_expert_ffn_arms_agree_with_oracle():
    g = torch.Generator().manual_seed(0)
    h, f, rows = 256, 192, 5
    x = torch.randn(rows, h, generator=g).to(torch.bfloat16)
    wgu = (torch.randn(2 * f, h, generator=g) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(h, f, generator=g) * 0.05).to(torch.bfloat16)
    want = ref.expert_ffn(x, wgu, wd, 0).float()
    outs = {}
    for arm in (0, 1, 2):
        try:
            outs[arm] = native.cpu_expert_ffn(x, wgu, wd, 0, arm).float()
        except RuntimeError:
            continue                            # this CPU lacks the arm
    assert 0 in outs
    for arm, y in outs.items():
        assert (y - want).abs().max() <= 2e-2 * want.abs().max() + 1e-3, f"arm {arm}"
    pool = native.ExpertPool(3)
    ys = [torch.empty(rows, h, dtype=torch.bfloat16) for _ in range(4)]
    pool.run([(x, wgu, wd, y) for y in ys])
    for y in ys:
        assert torch.equal(y, native.cpu_expert_ffn(x, wgu, wd))
    pool.close()


def test_direct_reader_unaligned_and_errors(tmp_path):
    data = os.urandom(3 * 4096 + 123)
    p = tmp_path / "blob.bin"
    p.write_bytes(data)
    rd = native.DirectReader(2)
    fd = rd.open(str(p))
    bufs, tickets = [], []
    for off, ln in ((0, 4096), (100, 5000), (4096 * 2 + 7, 4096 + 100), (len(data) - 10, 10)):
        b = torch.empty(ln, dtype=torch.uint8)
        tickets.append((rd.submit(fd, off, ln, b), off, ln, b))
    for t, off, ln, b in tickets:
        rd.wait(t)
        assert bytes(b.numpy().tobytes()) == data[off: off + ln]
    bad = rd.submit(fd, len(data) + 100000, 64, torch.empty(64, dtype=torch.uint8))
    with pytest.raises(OSError):
        rd.wait(bad)
    assert rd.in_flight() == 0
    rd.close()


@pytest.mark.parametrize("mode", ["score", "rank"])
def test_tiered_provider_matches_all_resident(mode):
    from flyingfish_b200.api import Model, generate_plain
    from flyingfish_b200.config import Settings
    from flyingfish_b200.experts.provider import build_provider_from_weights
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 2048, (24,), generator=g).tolist()
    m = Model.load("qwen3-moe-tiny", Settings(capacity=256, max_batch=2, graph=False), device="cpu", seed=0)
    plain = generate_plain(m, ids, 12, ignore_eos=True, graph=False).ids
    m.reset()
    prov = build_provider_from_weights(m.engine.model, resident_fraction=0.5, mode=mode, threads=2, admission_cap=2)
    assert sum(prov.cap.slots_per_layer) == prov.geo.total_experts // 2
    prov.collect_freq = True
    seq = m.engine.add_sequence(ids)
    first = m.engine.prefill([seq])[0]                    # cold slots: everything runs on the host pool
    prov.collect_freq = False
    prov.begin_request()                                 # install by prefill routing frequency
    for key in ("hits", "host_misses", "disk_misses"):
        prov.res.stats[key] = 0                          # measure the decode phase only
    out = [first] + [m.engine.decode([seq])[0] for _ in range(11)]
    agree = sum(a == b for a, b in zip(out, plain))
    assert agree >= 10, (out, plain)                     # FP32 SIMD vs FP64 oracle may flip a late token
    assert prov.stats["cpu_rows"] > 0 and prov.stats["gpu_rows"] > 0
    assert prov.res.stats["tokens"] == 11 and prov.res.hit_rate() > 0.3


def test_catalogue_disk_tier_and_span_plan(tmp_path):
    from flyingfish_b200.config import spec_from_hf_config
    from flyingfish_b200.experts.catalogue import ExpertCatalogue, slot_layout
    from flyingfish_b200.experts.disk import DiskExperts
    from flyingfish_b200.experts.span import ExpertClass, plan_layer
    from flyingfish_b200.loaders.checkpoint import manifest, save_decoder_checkpoint
    from flyingfish_b200.loaders.safetensors_io import MappedCheckpoint
    cfg = {"architectures": ["Qwen3MoeForCausalLM"], "hidden_size": 128, "num_attention_heads": 2, "num_key_value_heads": 1,
           "head_dim": 64, "intermediate_size": 256, "moe_intermediate_size": 64, "num_experts": 4, "num_experts_per_tok": 2,
           "num_hidden_layers": 2, "vocab_size": 256, "torch_dtype": "bfloat16", "hidden_act": "silu"}
    spec = spec_from_hf_config(cfg, "moe")
    g = torch.Generator().manual_seed(0)
    tensors = {n: (torch.randn(s, generator=g) * 0.05).to(torch.bfloat16) for n, (s, c) in manifest(spec).items()}
    d = tmp_path / "ck"
    save_decoder_checkpoint(d, spec, tensors, cfg, shards=2)
    ck = MappedCheckpoint(d)
    cat = ExpertCatalogue.from_checkpoint(ck, spec)
    lay = slot_layout(spec)
    assert cat.slot_bytes() == lay.total == 3 * 64 * 128 * 2 and len(cat.files()) == 2
    disk = DiskExperts(cat, {(1, 3), (0, 2)}, ring_slots=2, threads=2)
    assert disk.on_disk(1, 3) and not disk.on_disk(1, 0)
    disk.prefetch(0, [2])
    for (l, e) in ((1, 3), (0, 2), (1, 3)):
        gu, down = disk.fetch(l, e)
        p = f"model.layers.{l}.mlp.experts.{e}."
        assert torch.equal(gu[:64], tensors[p + "gate_proj.weight"]) and torch.equal(gu[64:], tensors[p + "up_proj.weight"])
        assert torch.equal(down, tensors[p + "down_proj.weight"])
    assert disk.stats["hits"] >= 1 and disk.stats["prefetched"] == 1
    disk.close(); ck.close()
    plan = plan_layer({0: 500, 1: 1, 2: 40, 3: 0}, resident={0}, slot_bytes=50_000_000, staging_slots=1,
                      rates=TransferRates(h2d_bytes_s=50e9), cpu=CpuService(per_expert_s=2e-4, workers=4))
    assert plan.classes[0] == ExpertClass.RESIDENT and plan.classes[2] == ExpertClass.STAGED
    assert plan.classes[1] == ExpertClass.CPU and 3 not in plan.classes
    assert [c.experts for c in plan.cohorts] == [[2]] and plan.cpu_rows == 1


def test_quantised_slot_layouts():
    """Slot layouts of the quantised expert formats: slice sizes, 16-byte alignment, pack / view round trip."""
    import torch
    from flyingfish_b200.experts.catalogue import FORMATS, pack_slot, quant_slot_layout, slot_views
    f, h = 96, 160
    sizes = {}
    for fmt in FORMATS:
        lay = quant_slot_layout(fmt, f, h)
        assert all(b % 16 == 0 for b, _ in lay.slices.values()) and lay.total % 16 == 0
        sizes[fmt] = lay.total
    assert sizes["bf16"] == sizes["bf16_separate"] == 3 * f * h * 2
    lay = quant_slot_layout("fp8_block", f, h)
    assert lay.code_bytes == 3 * f * h and lay.range("gate_scale")[1] - lay.range("gate_scale")[0] == 1 * 2 * 4
    assert lay.range("down_scale")[1] - lay.range("down_scale")[0] == 2 * 1 * 4
    assert quant_slot_layout("fp8_channel", f, h).scale_bytes == (f + f + h) * 4
    e2 = quant_slot_layout("e2m1_block", f, h)
    assert e2.code_bytes == 3 * f * h // 2 and e2.scale_bytes == 2 * f * (h // 32) + h * (f // 32)
    nv = quant_slot_layout("nvfp4", f, h)
    assert nv.scale_bytes == 2 * f * (h // 16) + h * (f // 16) + 12 and sizes["nvfp4"] < sizes["fp8_block"] < sizes["bf16"]
    with pytest.raises(ValueError):
        quant_slot_layout("e2m1_block", 100, 160)
    g = torch.Generator().manual_seed(0)
    t = {n: torch.randint(0, 255, (e - b,), generator=g, dtype=torch.uint8) for n, (b, e) in e2.slices.items()}
    views = slot_views(e2, pack_slot(e2, t))
    assert views["gate"].shape == (f, h // 2) and views["down_scale"].shape == (h, f // 32)
    assert torch.equal(views["up"].reshape(-1), t["up"]) and torch.equal(views["gate_scale"].reshape(-1), t["gate_scale"])
    fb = quant_slot_layout("fp8_block", 256, 384)
    tb = {n: torch.randint(0, 255, (e - b,), generator=g, dtype=torch.uint8) for n, (b, e) in fb.slices.items()}
    vb = slot_views(fb, pack_slot(fb, tb))
    assert vb["gate_scale"].shape == (2, 3) and vb["down_scale"].shape == (3, 2) and vb["gate"].shape == (256, 384)
