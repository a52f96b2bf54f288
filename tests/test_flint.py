"""Flint-style decoder: learnable soft-max (attention sinks), local layers with a window and rotary positions, global
layers without positions. The sink arithmetic against a direct soft-max, chunked prefill against decode on the CPU
oracles, and the CUDA kernels / model against the CPU."""
import pytest
import torch

from flyingfish_b200 import ops
from flyingfish_b200.api import Model
from flyingfish_b200.config import Settings


def _attn_case(seed=0, hq=4, hkv=1, d=128, ctx=150, nb=8):
    g = torch.Generator().manual_seed(seed)
    kc = torch.randn(nb, hkv, 64, d, generator=g).to(torch.bfloat16)
    vc = torch.randn(nb, hkv, 64, d, generator=g).to(torch.bfloat16)
    bt = torch.tensor([[2, 5, 1, 0]], dtype=torch.int32)
    q = torch.randn(1, (hq + 2 * hkv) * d, generator=g).to(torch.bfloat16)
    sinks = torch.randn(hq, generator=g) * 2
    return q, kc, vc, bt, torch.tensor([ctx], dtype=torch.int32), sinks


def test_sink_is_an_extra_logit_without_a_value():
    q, kc, vc, bt, cl, sinks = _attn_case()
    hq, hkv, d = 4, 1, 128
    out = ops.attn_decode(q, kc, vc, bt, cl, hq, hkv, d, d ** -0.5, sinks=sinks).float().view(hq, d)
    base = ops.attn_decode(q, kc, vc, bt, cl, hq, hkv, d, d ** -0.5).float().view(hq, d)
    # with the sink the output is the plain output scaled by (1 - sink probability) per head
    k = torch.cat([kc[2, 0], kc[5, 0], kc[1, 0]])[:150].float()
    s = (q[0, : hq * d].float().view(hq, d) @ k.t()) * d ** -0.5
    psink = torch.softmax(torch.cat([s, sinks[:, None]], 1), 1)[:, -1]
    assert torch.allclose(out, base * (1 - psink)[:, None], atol=2e-2)
    huge = ops.attn_decode(q, kc, vc, bt, cl, hq, hkv, d, d ** -0.5, sinks=torch.full((hq,), 60.0)).float()
    assert huge.abs().max() < 1e-3


def _load(device, **kw):
    return Model.load("flint-tiny", Settings(capacity=512, max_batch=4, graph=False, **kw), device=device, seed=0)


def _prompts():
    g = torch.Generator().manual_seed(5)
    return [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (90, 12)]


def test_flint_chunked_prefill_and_decode_agree_cpu():
    from _oracle import assert_tokens_equal_up_to_ties
    p = _prompts()
    m = _load("cpu")
    net = m.engine.model
    assert net.window == 33 and sorted(net.no_rope) == [0, 1, 4] and len(net.sinks) == 5
    want = m.generate_batch(p, 8)
    got = _load("cpu", chunk=32).generate_batch(p, 8)
    for pr, w, g in zip(p, want, got):
        assert_tokens_equal_up_to_ties(m, pr, w, g)
    nxt = _load("cpu").generate_batch([p[0] + want[0][:4]], 1)[0][0]
    assert nxt == want[0][4]


@pytest.mark.gpu
def test_sink_attention_cuda_matches_oracle():
    hq, hkv, d = 8, 2, 128
    g = torch.Generator().manual_seed(3)
    nb = 40
    kc = torch.randn(nb, hkv, 64, d, generator=g).to(torch.bfloat16)
    vc = torch.randn(nb, hkv, 64, d, generator=g).to(torch.bfloat16)
    sinks = torch.randn(hq, generator=g) * 2
    lens = [700, 64, 1300]
    bt = torch.zeros(3, 24, dtype=torch.int32)
    perm = torch.randperm(nb, generator=g)
    at = 0
    for i, n in enumerate(lens):
        nblk = (n + 63) // 64
        bt[i, :nblk] = (perm[torch.arange(nblk) % nb] if nblk > nb - at else perm[at: at + nblk]).to(torch.int32)
        at = (at + nblk) % (nb - 24)
    cl = torch.tensor(lens, dtype=torch.int32)
    q = torch.randn(3, (hq + 2 * hkv) * d, generator=g).to(torch.bfloat16)
    for window in (0, 100):
        want = ops.attn_decode(q, kc, vc, bt, cl, hq, hkv, d, d ** -0.5, window=window, sinks=sinks)
        got = ops.attn_decode(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), cl.cuda(), hq, hkv, d, d ** -0.5, window=window,
                              sinks=sinks.cuda(), max_ctx=1536)
        assert (got.cpu().float() - want.float()).abs().max() < 2e-2, window
    # prefill: two sequences, chunk rows against the whole context
    q_lens = torch.tensor([200, 64], dtype=torch.int32); ctx = torch.tensor([700, 64], dtype=torch.int32)
    q_start = torch.tensor([0, 200], dtype=torch.int32)
    qp = torch.randn(264, (hq + 2 * hkv) * d, generator=g).to(torch.bfloat16)
    for window in (0, 100):
        want = ops.attn_prefill(qp, kc, vc, bt[:2], q_start, q_lens, ctx, 200, hq, hkv, d, d ** -0.5, window=window, sinks=sinks)
        got = ops.attn_prefill(qp.cuda(), kc.cuda(), vc.cuda(), bt[:2].cuda().contiguous(), q_start.cuda(), q_lens.cuda(), ctx.cuda(), 200,
                               hq, hkv, d, d ** -0.5, window=window, sinks=sinks.cuda())
        assert (got.cpu().float() - want.float()).abs().max() < 3e-2, window
    ops.check_status()


@pytest.mark.gpu
def test_flint_model_gpu_matches_cpu_oracle():
    from _oracle import assert_tokens_equal_up_to_ties
    p = _prompts()
    cpu, gpu = _load("cpu"), _load("cuda")
    want, got = cpu.generate_batch(p, 8), gpu.generate_batch(p, 8)
    ops.check_status()
    for pr, w, g in zip(p, want, got):
        assert_tokens_equal_up_to_ties(cpu, pr, w, g)
    graphs = Model.load("flint-tiny", Settings(capacity=512, max_batch=4, graph=True), device="cuda", seed=0)
    assert graphs.generate_batch(p, 8) == got and graphs.engine.stats["graph_replays"] > 0
