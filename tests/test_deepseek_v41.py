"""DeepSeek-V4.1-style model (hyper-connection streams, latent window ring, top-k sparse layer with a pooled indexer,
Engram rows, square-root-soft-plus routing): consistency of chunked prefill and decoding on the CPU oracle operators,
the new operators against their oracles on the GPU, and the GPU model against the CPU model."""
import pytest
import torch

from flyingfish_b200.api import Model
from flyingfish_b200.config import Settings
from flyingfish_b200.ops import dsa_ops, latent_ops as lo, moe_ops, ref

NAME = "deepseek-v41-tiny"


def _prompts(lens, seed=3):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, 2048, (n,), generator=g).tolist() for n in lens]


def _load(device="cpu", **kw):
    return Model.load(NAME, Settings(capacity=256, max_batch=4, graph=False, **kw), device=device, seed=0)


def test_prefill_chunks_and_decode_agree_on_cpu():
    """One 70-token prompt (longer than the 32-token window, 17 pools for the sparse layer): a prefill in chunks of 16
    rows, a prefill in one chunk, and token-by-token decoding of the continuation must tell the same story."""
    from _oracle import assert_tokens_equal_up_to_ties
    p = _prompts([70, 9])
    whole = _load()
    want = whole.generate_batch(p, 8)
    chunked = _load(chunk=16)
    assert chunked.engine.model.ring == 32 + 16 - 1 and whole.engine.model.ring == 32 + 256 - 1
    got = chunked.generate_batch(p, 8)
    for pr, w, g in zip(p, want, got):
        assert_tokens_equal_up_to_ties(whole, pr, w, g)
    # decode rows continue exactly what a prefill of the longer prompt computes
    again = _load()
    nxt = again.generate_batch([p[0] + want[0][:5]], 1)[0][0]
    assert nxt == want[0][5]
    st = whole.engine.model.engram["services"][0].stats
    assert st["hits"] + st["misses"] > 0                   # the n-gram memory rows were served


def test_window_layers_forget_and_sparse_layer_remembers():
    """Changing a token far outside the window changes the output (the sparse layer, the hyper-connection streams and
    the n-gram rows carry it), while the window ring itself only holds the last ``window`` positions."""
    m = _load()
    p = _prompts([80])[0]
    m.generate_batch([p], 1)
    net = m.engine.model
    assert all(c.shape[1] == net.ring for c in net.codes.values()) and net.window == 32
    assert sorted(net.sparse_layers) == [1] and net.pooled[1].abs().sum() > 0


def test_glm_style_shape_all_sparse_layers_cpu():
    """GLM-style variant: own pre-mix at every stage, sparse attention in all layers, no window ring, no n-gram rows."""
    m = Model.load("glm5-next-tiny", Settings(capacity=256, max_batch=4, graph=False), device="cpu", seed=0)
    net = m.engine.model
    assert net.hc_policy == "own" and not net.codes and sorted(net.sparse_layers) == [0, 1, 2] and net.engram is None
    p = _prompts([45])
    want = m.generate_batch(p, 6)
    again = Model.load("glm5-next-tiny", Settings(capacity=256, max_batch=4, graph=False, chunk=16), device="cpu", seed=0)
    from _oracle import assert_tokens_equal_up_to_ties
    assert_tokens_equal_up_to_ties(m, p[0], want[0], again.generate_batch(p, 6)[0])


def test_router_sqrt_softplus_oracle():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 64, generator=g).to(torch.bfloat16)
    w = (torch.randn(16, 64, generator=g) * 0.3).to(torch.bfloat16)
    bias = torch.randn(16, generator=g) * 0.1
    wt, ids = ref.moe_route(x, w, 4, "sqrt_softplus", bias, 1, 1, 2.0, True)
    logits = (x.float() @ w.float().t()).to(torch.bfloat16).float()
    s = torch.sqrt(torch.nn.functional.softplus(logits))
    top = torch.topk(s + bias, 4).indices
    assert set(ids[0].tolist()) == set(top[0].tolist())
    assert torch.allclose(wt.sum(-1), torch.full((5,), 2.0), atol=1e-5)


def test_state_checkpoint_roundtrip_cpu():
    tabs = [torch.randn(40, 64).to(torch.bfloat16), torch.randn(40, 128).to(torch.bfloat16)]
    keep = [t.clone() for t in tabs]
    rows = torch.tensor([3, 17, 39], dtype=torch.int32)
    snap = dsa_ops.checkpoint_save(tabs, rows)
    for t in tabs:
        t[rows.long()] = 0
    dsa_ops.checkpoint_restore(snap)
    assert all(torch.equal(a, b) for a, b in zip(tabs, keep))


@pytest.mark.gpu
def test_new_operators_cuda_match_oracles():
    from flyingfish_b200 import ops
    g = torch.Generator().manual_seed(1)
    # pair rotary on the tail
    rows, heads, d, tail = 37, 4, 128, 32
    x = torch.randn(rows, heads * d, generator=g).to(torch.bfloat16)
    pos = torch.randint(0, 500, (rows,), generator=g).to(torch.int32)
    cs = lo.rotary_table(pos, tail, 1e4)
    want = x.clone(); lo.rope_pair_tail(want, cs, heads, d, tail)
    got = x.cuda(); lo.rope_pair_tail(got, cs.cuda(), heads, d, tail)
    assert torch.equal(want[:, : d - tail], x[:, : d - tail]) and not torch.equal(want, x)
    assert (got.cpu().float() - want.float()).abs().max() <= 2e-2
    back = got.clone(); lo.rope_pair_tail(back, lo.rotary_table(pos, tail, 1e4, inverse=True).cuda(), heads, d, tail)
    assert (back.cpu().float() - x.float()).abs().max() <= 4e-2
    # window shorter than the ring: prefill rows of one sequence as independent queries
    ring, window, n = 47, 32, 60
    codes = torch.zeros(2, ring, d, dtype=torch.uint8); scales = torch.full((2, ring, d // 32), 127, dtype=torch.uint8)
    k = (torch.randn(n, d, generator=g) * 1.5).to(torch.bfloat16)
    q = torch.randn(16, heads, d, generator=g).to(torch.bfloat16)
    sink = torch.randn(heads, generator=g)
    qpos = torch.arange(n - 16, n, dtype=torch.int32)
    rid = torch.ones(16, dtype=torch.int32)
    # positions 0..n-17 arrive one launch earlier; the last 16 rows are one chunk written before their queries run
    lo.ring_write(k[: n - 16], torch.ones(n - 16, dtype=torch.int32), torch.arange(n - 16, dtype=torch.int32), codes, scales)
    lo.ring_write(k[n - 16:], rid, qpos, codes, scales)
    want = lo.window_attention(q, codes, scales, rid, qpos, sink, tail, 1e4, visible=window)
    got = lo.window_attention(q.cuda(), codes.cuda(), scales.cuda(), rid.cuda(), qpos.cuda(), sink.cuda(), tail, 1e4,
                              visible=window)
    assert (got.cpu().float() - want.float()).abs().max() <= 3e-2
    # the oracle itself: row j sees exactly positions qpos[j]-31 .. qpos[j]
    full = torch.zeros(1, n, d, dtype=torch.uint8); fs = torch.full((1, n, d // 32), 127, dtype=torch.uint8)
    lo.ring_write(k, torch.zeros(n, dtype=torch.int32), torch.arange(n, dtype=torch.int32), full, fs)
    for j in (0, 7, 15):
        p = int(qpos[j])
        lone = lo.window_attention(q[j: j + 1], full[:, p - 31: p + 1].contiguous(), fs[:, p - 31: p + 1].contiguous(),
                                   torch.zeros(1, dtype=torch.int32), torch.tensor([31], dtype=torch.int32), sink, 0, 1e4)
        ref_row = lo.window_attention(q[j: j + 1], codes, scales, rid[:1], qpos[j: j + 1], sink, 0, 1e4, visible=window)
        assert torch.equal(lone, ref_row)
    # router
    xr = torch.randn(33, 256, generator=g).to(torch.bfloat16); wr = (torch.randn(8, 256, generator=g) * 0.2).to(torch.bfloat16)
    bias = torch.randn(8, generator=g) * 0.05
    w0, i0 = moe_ops.route(xr, wr, 2, "sqrt_softplus", bias, 1, 1, 1.5, True)
    w1, i1 = moe_ops.route(xr.cuda(), wr.cuda(), 2, "sqrt_softplus", bias.cuda(), 1, 1, 1.5, True)
    same = (i0 == i1.cpu()).all(dim=1)
    assert same.float().mean() > 0.9 and torch.allclose(w0[same], w1.cpu()[same], atol=2e-2)
    # checkpoint of state rows
    tabs = [torch.randn(50, 128, generator=g).to(torch.bfloat16).cuda(), torch.randn(50, 64, generator=g).to(torch.bfloat16).cuda(),
            torch.randint(0, 255, (50, 48), generator=g).to(torch.uint8).cuda()]
    keep = [t.clone() for t in tabs]
    sel = torch.tensor([0, 13, 49, 20], dtype=torch.int32).cuda()
    snap = dsa_ops.checkpoint_save(tabs, sel)
    for t in tabs:
        t[sel.long()] = 0
    assert not torch.equal(tabs[0], keep[0])
    dsa_ops.checkpoint_restore(snap)
    assert all(torch.equal(a, b) for a, b in zip(tabs, keep))
    ops.check_status()


@pytest.mark.gpu
def test_v41_model_gpu_matches_cpu_oracle():
    from _oracle import assert_rows_mostly_close, assert_tokens_equal_up_to_ties
    from flyingfish_b200 import ops
    p = _prompts([70, 9])
    cpu, gpu = _load(), _load("cuda")
    want, got = cpu.generate_batch(p, 8), gpu.generate_batch(p, 8)
    ops.check_status()
    for pr, w, g in zip(p, want, got):
        assert_tokens_equal_up_to_ties(cpu, pr, w, g)
    chunked = _load("cuda", chunk=16).generate_batch(p, 8)
    for pr, w, g in zip(p, want, chunked):
        assert_tokens_equal_up_to_ties(cpu, pr, w, g)
    st = Settings(capacity=256, max_batch=4, graph=False)
    c2, g2 = (Model.load("glm5-next-tiny", st, device=d, seed=0) for d in ("cpu", "cuda"))
    for pr, w, g in zip(p, c2.generate_batch(p, 8), g2.generate_batch(p, 8)):
        assert_tokens_equal_up_to_ties(c2, pr, w, g)
    ops.check_status()
