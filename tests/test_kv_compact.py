"""Paged 8-bit KV store (``--kv-format affine8``): sealing of old groups, block release, and decode attention over
sink + sealed groups + recent pages against the BF16 cache."""
import pytest
import torch

from flyingfish_b200.api import Model
from flyingfish_b200.config import Settings
from flyingfish_b200.engine.kv_compact import CompactKV, sealed_until


def test_sealed_boundary():
    assert sealed_until(2048 + 127) == 0 and sealed_until(2048 + 128) == 128 and sealed_until(500, recent=128) == 256
    assert CompactKV.bytes_per_slot(1, 1, 128) == 2 * 128 * 128 + 128 * 8 + 128 * 8          # vs 65 536 bytes in BF16


def _models(device, recent=128, capacity=1024):
    a = Model.load("tiny-llama", Settings(capacity=capacity, max_batch=4, graph=False), device=device, seed=0)
    b = Model.load("tiny-llama", Settings(capacity=capacity, max_batch=4, graph=False, kv_format="affine8",
                                          kv_recent=recent), device=device, seed=0)
    return a, b


def _prompts():
    g = torch.Generator().manual_seed(11)
    return [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (420, 70)]


def test_sealing_releases_blocks_and_decode_tracks_bf16_cpu():
    plain, packed = _models("cpu")
    p = _prompts()
    want = plain.generate_batch(p, 24)
    eng = packed.engine
    seqs = [eng.add_sequence(x) for x in p]
    free0 = eng.kv.alloc.free_blocks
    eng.prefill(seqs)
    got = [[s.output[0]] for s in seqs]
    for _ in range(23):
        for s, t in zip(seqs, eng.decode(seqs)):
            got[seqs.index(s)].append(t)
    c = eng.kv.compact
    long, short = seqs
    # 420 + 24 tokens, recent 128: groups [0, 2) sealed at least (positions < 256), the short sequence has none
    assert c.sealed_tokens(long.seq_id) == sealed_until(eng.kv.seqs[long.seq_id].length, 128) >= 256
    assert c.sealed_tokens(short.seq_id) == 0
    blocks = eng.kv.seqs[long.seq_id].blocks
    ng = c.sealed_tokens(long.seq_id) // 128
    assert blocks[0] >= 0 and all(b == -1 for b in blocks[1: 2 * ng]) and all(b >= 0 for b in blocks[2 * ng:])
    assert c.stats["released_blocks"] == 2 * ng - 1
    # 8-bit rows perturb logits a little: the greedy continuations agree at the start and the short sequence exactly
    assert got[1] == want[1]
    agree = next((i for i, (a, b) in enumerate(zip(want[0], got[0])) if a != b), 24)
    assert agree >= 6, (want[0], got[0])
    used = free0 - eng.kv.alloc.free_blocks
    for s in seqs:
        eng.free_sequence(s.seq_id)
    assert eng.kv.alloc.free_blocks == free0 and c.free_slots == c.slots and used > 0
    with pytest.raises(ValueError):
        eng.verify([eng.add_sequence([1, 2, 3])], [[4]])


def test_attention_over_sealed_groups_matches_materialised_oracle():
    """The mixed decode attention equals attention over the dequantised rows (the CPU path is that oracle), and the
    dequantised rows are within one code step of the originals."""
    from flyingfish_b200 import ops
    from flyingfish_b200.engine.kv_cache import PagedKVCache
    g = torch.Generator().manual_seed(2)
    hkv, hq, d, nb = 2, 8, 128, 16
    kv = PagedKVCache(1, hkv, d, nb, 64, torch.bfloat16, "cpu")
    kv.k[0].copy_(torch.randn(nb, hkv, 64, d, generator=g).to(torch.bfloat16))
    kv.v[0].copy_(torch.randn(nb, hkv, 64, d, generator=g).to(torch.bfloat16))
    keep = (kv.k[0].clone(), kv.v[0].clone())
    s = kv.add_sequence(0)
    kv.reserve(0, 700); kv.commit(0, 700)
    blocks0 = list(s.blocks)
    c = CompactKV(1, hkv, d, 8, "cpu", recent=128)
    kv.compact = c
    assert c.seal(kv, 0) == 4                                   # sealed_until(700, 128) = 512 tokens = 4 groups
    kd, vd = c.dequant(0, c.groups[0][1])
    ref_k = torch.cat([keep[0][blocks0[2]], keep[0][blocks0[3]]], dim=1).float()
    span = ref_k.amax(1, keepdim=True) - ref_k.amin(1, keepdim=True)
    assert ((kd.float() - ref_k).abs() <= span / 255 * 0.51 + 0.02).all()
    q = torch.randn(1, (hq + 2 * hkv) * d, generator=g).to(torch.bfloat16)
    bt = torch.tensor([[b if b >= 0 else 0 for b in s.blocks] + [0] * 4], dtype=torch.int32)
    gt = torch.tensor([c.groups[0] + [0] * 4], dtype=torch.int32)
    out = ops.attn_decode_mixed(q, kv.k[0], kv.v[0], c, 0, bt, torch.tensor([700], dtype=torch.int32),
                                torch.tensor([512], dtype=torch.int32), gt, hq, hkv, d, d ** -0.5)
    full_bt = torch.tensor([blocks0 + [0] * 4], dtype=torch.int32)
    want = ops.attn_decode(q, keep[0], keep[1], full_bt, torch.tensor([700], dtype=torch.int32), hq, hkv, d, d ** -0.5)
    assert (out.float() - want.float()).abs().max() < 0.03


@pytest.mark.gpu
def test_mixed_decode_attention_cuda_matches_cpu_oracle():
    from flyingfish_b200 import ops
    from flyingfish_b200.engine.kv_cache import PagedKVCache
    g = torch.Generator().manual_seed(3)
    hkv, hq, d, nb, batch = 2, 8, 128, 64, 3
    kc = torch.randn(nb, hkv, 64, d, generator=g).to(torch.bfloat16)
    vc = torch.randn(nb, hkv, 64, d, generator=g).to(torch.bfloat16)
    res = {}
    for dev in ("cpu", "cuda"):
        kv = PagedKVCache(1, hkv, d, nb, 64, torch.bfloat16, dev)
        kv.k[0].copy_(kc); kv.v[0].copy_(vc)
        c = CompactKV(1, hkv, d, 24, dev, recent=128)
        kv.compact = c
        lens = [900, 130, 1290]
        rows, groups = [], []
        for i, n in enumerate(lens):
            kv.add_sequence(i); kv.reserve(i, n); kv.commit(i, n)
            c.seal(kv, i)
            rows.append([b if b >= 0 else 0 for b in kv.seqs[i].blocks]); groups.append(list(c.groups[i]))
        width = 24
        bt = torch.tensor([r + [0] * (width - len(r)) for r in rows], dtype=torch.int32, device=dev)
        gt = torch.tensor([r + [0] * (12 - len(r)) for r in groups], dtype=torch.int32, device=dev)
        ks = torch.tensor([len(r) * 128 for r in groups], dtype=torch.int32, device=dev)
        q = torch.randn(batch, (hq + 2 * hkv) * d, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16).to(dev)
        res[dev] = ops.attn_decode_mixed(q, kv.k[0], kv.v[0], c, 0, bt, torch.tensor(lens, dtype=torch.int32, device=dev), ks, gt,
                                         hq, hkv, d, d ** -0.5).float().cpu()
        res[dev + "_codes"] = (c.k_codes[0].cpu(), c.v_codes[0].cpu(), c.k_stats[0].cpu(), c.v_stats[0].cpu(), ks.cpu())
    ops.check_status()
    assert res["cpu_codes"][4].tolist() == [768, 0, 1152]
    for a, b in zip(res["cpu_codes"][:4], res["cuda_codes"][:4]):           # the seal kernel packs the same codes and statistics
        assert torch.equal(a, b) if a.dtype == torch.uint8 else torch.allclose(a, b, rtol=0, atol=0)
    assert (res["cpu"] - res["cuda"]).abs().max() < 0.02


@pytest.mark.gpu
def test_affine8_model_decodes_on_gpu_with_graphs():
    plain = Model.load("tiny-llama", Settings(capacity=1024, max_batch=4, graph=True), device="cuda", seed=0)
    packed = Model.load("tiny-llama", Settings(capacity=1024, max_batch=4, graph=True, kv_format="affine8", kv_recent=128),
                        device="cuda", seed=0)
    p = _prompts()
    want, got = plain.generate_batch(p, 24), packed.generate_batch(p, 24)
    from flyingfish_b200 import ops
    ops.check_status()
    assert got[1] == want[1]
    agree = next((i for i, (a, b) in enumerate(zip(want[0], got[0])) if a != b), 24)
    assert agree >= 6, (want[0], got[0])
    assert packed.engine.kv.compact.stats["sealed_groups"] >= 2 and packed.engine.stats["graph_replays"] > 0
