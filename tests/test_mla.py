"""Multi-head latent attention: CPU model invariants and the CUDA kernel against the oracle."""
import math

import pytest
import torch

from flyingfish_b200.api import Model, generate_plain
from flyingfish_b200.config import Settings


@pytest.mark.parametrize("name", ["deepseek-v3-tiny", "deepseek-v3-mini"])
def test_deepseek_cpu_chunk_and_batch_invariance(name):
    m = Model.load(name, Settings(capacity=256, max_batch=4, graph=False), device="cpu", seed=0)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, m.spec.vocab, (30,), generator=g).tolist()
    a = generate_plain(m, ids, 5, ignore_eos=True).ids
    m.reset(); m.settings.chunk = 9
    assert generate_plain(m, ids, 5, ignore_eos=True).ids == a
    m.reset(); m.settings.chunk = None
    assert m.generate_batch([ids, ids[:7]], 5)[0] == a
    assert m.engine.kv.k[0].shape[-1] == m.spec.mla.kv_lora_rank + m.spec.mla.qk_rope_dim and m.engine.kv.v[0] is None


@pytest.mark.gpu
@pytest.mark.parametrize("heads,qlens,pasts", [(4, [1, 1, 1], [0, 63, 200]), (128, [1], [700]), (4, [70, 5], [0, 100]),
                                               (16, [33], [64])])
def test_mla_attention_kernel(heads, qlens, pasts):
    from flyingfish_b200 import ops
    from flyingfish_b200.ops import mla_ops
    g = torch.Generator().manual_seed(3)
    batch = len(qlens)
    max_blocks = 16
    cache = torch.randn(batch * max_blocks, 1, 64, 576, generator=g).to(torch.bfloat16)
    bt = torch.randperm(batch * max_blocks, generator=g).to(torch.int32).view(batch, max_blocks)
    ql = torch.tensor(qlens, dtype=torch.int32)
    qs = (torch.cumsum(ql, 0) - ql).to(torch.int32)
    ctx = ql + torch.tensor(pasts, dtype=torch.int32)
    rows = int(ql.sum())
    q = (torch.randn(rows, heads, 576, generator=g) * 0.3).to(torch.bfloat16)
    scale = 1 / math.sqrt(192)
    want = mla_ops.attention(q, cache, bt, qs, ql, ctx, max(qlens), int(ctx.max()), scale, 512).float()
    got = mla_ops.attention(q.cuda(), cache.cuda(), bt.cuda(), qs.cuda(), ql.cuda(), ctx.cuda(), max(qlens),
                            int(ctx.max()), scale, 512)
    torch.cuda.synchronize()
    ops.check_status()
    err = (got.float().cpu() - want).abs()
    assert (err <= 2e-2 + 2e-2 * want.abs()).all(), f"max err {err.max().item()}"


@pytest.mark.gpu
def test_deepseek_mini_gpu_eager_graph_and_cpu_agreement():
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, 2048, (45,), generator=g).tolist()
    m = Model.load("deepseek-v3-mini", Settings(capacity=256, max_batch=4), device="cuda", seed=0)
    a = generate_plain(m, ids, 8, ignore_eos=True, graph=False).ids
    m.reset()
    b = generate_plain(m, ids, 8, ignore_eos=True, graph=True).ids
    assert a == b
    m.reset(); m.settings.chunk = 64
    long_ids = torch.randint(0, 2048, (150,), generator=g).tolist()
    c1 = generate_plain(m, long_ids, 4, ignore_eos=True, graph=False).ids
    m.reset(); m.settings.chunk = None
    assert generate_plain(m, long_ids, 4, ignore_eos=True, graph=False).ids == c1


@pytest.mark.gpu
def test_tiered_experts_on_gpu():
    from flyingfish_b200.experts.provider import build_provider_from_weights
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, 2048, (24,), generator=g).tolist()
    m = Model.load("qwen3-moe-tiny", Settings(capacity=256, max_batch=2, graph=False), device="cuda", seed=0)
    plain = generate_plain(m, ids, 10, ignore_eos=True, graph=False).ids
    m.reset()
    prov = build_provider_from_weights(m.engine.model, resident_fraction=0.5, threads=2, admission_cap=2)
    prov.collect_freq = True
    seq = m.engine.add_sequence(ids)
    first = m.engine.prefill([seq])[0]
    prov.collect_freq = False
    prov.begin_request()
    out = [first] + [m.engine.decode([seq])[0] for _ in range(9)]
    assert sum(x == y for x, y in zip(out, plain)) >= 8, (out, plain)
    assert prov.stats["cpu_rows"] > 0 and prov.stats["gpu_rows"] > 0 and prov.stats["h2d_expert_bytes"] > 0
