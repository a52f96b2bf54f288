"""Numerics of every CUDA operator against the plain PyTorch FP32 oracle of the same op."""
import math

import pytest
import torch

from flyingfish_b200 import ops
from flyingfish_b200.ops import ref

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _rand(shape, seed, scale=1.0, device="cuda"):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(BF16).to(device)


def _close(a, b, rtol=2e-2, atol=2e-2):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = (err > tol).sum().item()
    assert bad == 0, f"{bad} / {a.numel()} mismatches, max err {err.max().item():.4g}"


@pytest.mark.parametrize("m,n,k", [(1, 256, 64), (16, 384, 128), (64, 4096, 4096), (128, 1024, 512),
                                   (7, 6144, 4096), (33, 128256 // 8, 1024)])
def test_gemm_skinny(m, n, k):
    x, w = _rand((m, k), 1), _rand((n, k), 2, 0.05)
    y = ops.linear(x, w)
    torch.cuda.synchronize()
    ops.check_status()
    _close(y, ref.linear(x.cpu(), w.cpu()))


@pytest.mark.parametrize("m,n,k", [(129, 256, 64), (256, 512, 256), (1000, 768, 320), (2048, 4096, 4096),
                                   (300, 1000, 136)])
def test_gemm_large(m, n, k):
    x, w = _rand((m, k), 3), _rand((n, k), 4, 0.05)
    y = ops.linear(x, w)
    torch.cuda.synchronize()
    ops.check_status()
    _close(y, ref.linear(x.cpu(), w.cpu()))


def test_gemm_fp32_out():
    x, w = _rand((200, 256), 5), _rand((512, 256), 6, 0.05)
    y = ops.linear(x, w, out_dtype=torch.float32)
    ops.check_status()
    _close(y, x.float().cpu() @ w.float().cpu().t(), 1e-3, 1e-3)


def test_gemm_deterministic_and_repeatable():
    x, w = _rand((48, 4096), 7), _rand((4096, 4096), 8, 0.05)
    a = ops.linear(x, w).clone()
    b = ops.linear(x, w).clone()
    assert torch.equal(a, b)


@pytest.mark.parametrize("m", [8, 300])
def test_gemm_swiglu(m):
    f, h = 512, 256
    x = _rand((m, h), 9)
    wg, wu = _rand((f, h), 10, 0.05), _rand((f, h), 11, 0.05)
    wi = ref.interleave_gate_up(wg, wu)
    y = ops.linear_swiglu(x, wi)
    ops.check_status()
    expect = ref.silu_mul(torch.cat([ref.linear(x.cpu(), wg.cpu()), ref.linear(x.cpu(), wu.cpu())], dim=1))
    _close(y, expect)


@pytest.mark.parametrize("m,f,h", [(64, 14336, 1024), (7, 1024, 4096), (128, 2048, 512)])
def test_decode_gemm_swiglu_epilogue_matches_unfused(m, f, h):
    """The decode GEMM's SwiGLU epilogue (stream-K and cluster split-K decompositions) against GEMM
    followed by the stand-alone activation kernel. The two GEMMs may split K differently (the fused
    one uses 128-row tiles), so sums can differ in the last FP32 bit before rounding."""
    x = _rand((m, h), 31)
    wi = ref.interleave_gate_up(_rand((f, h), 32, 0.05), _rand((f, h), 33, 0.05))
    fused = ops.linear_swiglu(x, wi)
    unfused = ops.silu_mul_interleaved(ops.linear(x, wi))
    ops.check_status()
    _close(fused, unfused, 2e-2, 2e-2)
    assert torch.equal(fused, ops.linear_swiglu(x, wi))


@pytest.mark.parametrize("m,hq,hkv,h", [(64, 32, 8, 1024), (5, 4, 2, 4096), (128, 16, 16, 512)])
def test_decode_gemm_rope_kv_epilogue_matches_unfused(m, hq, hkv, h):
    d, bs, nb = 128, 64, 8
    x = _rand((m, h), 34)
    w = _rand(((hq + 2 * hkv) * d, h), 35, 0.05)
    pos = torch.arange(50, 50 + m, dtype=torch.int32, device="cuda")
    slots = (torch.arange(m, dtype=torch.int32) + 9).to("cuda")
    slots[min(3, m - 1)] = -1
    kc = torch.zeros(nb, hkv, bs, d, dtype=BF16, device="cuda"); vc = torch.zeros_like(kc)
    kc2, vc2 = kc.clone(), vc.clone()
    fused = ops.linear_rope_kv(x, w, pos, slots, kc, vc, hq, hkv, d, 5e5)
    qkv = ops.linear(x, w)
    ops.rope_kv_paged(qkv, pos, slots, kc2, vc2, hq, hkv, d, 5e5)
    ops.check_status()
    _close(fused, qkv, 2e-2, 2e-2)
    _close(kc, kc2, 2e-2, 2e-2)
    _close(vc, vc2, 2e-2, 2e-2)


@pytest.mark.parametrize("rows,hidden", [(1, 4096), (64, 4096), (5, 7168), (3, 256), (2, 8192)])
def test_norms(rows, hidden):
    x, res, w = _rand((rows, hidden), 12), _rand((rows, hidden), 13), _rand((hidden,), 14)
    n = ops.rmsnorm(x, w, 1e-5)
    _close(n, ref.rmsnorm(x.cpu(), w.cpu(), 1e-5), 1e-2, 1e-2)
    res2 = res.clone()
    n2 = ops.add_rmsnorm(x, res2, w, 1e-5)
    er, en = ref.add_rmsnorm(x.cpu(), res.cpu(), w.cpu(), 1e-5)
    assert torch.equal(res2.cpu(), er), "residual must be bit-exact (one BF16 rounding of the sum)"
    _close(n2, en, 1e-2, 1e-2)
    ops.check_status()


def test_embed_rmsnorm_and_bad_id_status():
    vocab, hidden = 1000, 512
    table, w = _rand((vocab, hidden), 15), _rand((hidden,), 16)
    ids = torch.tensor([0, 5, 999, 17], dtype=torch.int32, device="cuda")
    x, n = ops.embed_rmsnorm(ids, table, w, 1e-6)
    ex, en = ref.embed_rmsnorm(ids.cpu(), table.cpu(), w.cpu(), 1e-6)
    assert torch.equal(x.cpu(), ex)
    _close(n, en, 1e-2, 1e-2)
    ops.check_status()
    # a token id outside the table is reported through the status word, not by a fault
    bad = torch.tensor([3, 1000], dtype=torch.int32, device="cuda")
    ops.embed_rmsnorm(bad, table, w, 1e-6)
    code, kid, d0, d1 = ops.read_status()
    assert code == 3 and d0 == 1 and d1 == 1000
    assert ops.read_status()[0] == 0


def test_rope_kv_paged():
    rows, hq, hkv, d, bs, nb = 37, 4, 2, 128, 64, 6
    qkv = _rand((rows, (hq + 2 * hkv) * d), 17)
    pos = torch.arange(100, 100 + rows, dtype=torch.int32, device="cuda")
    slots = (torch.arange(rows, dtype=torch.int32) + 70).to("cuda")
    slots[3] = -1
    kc = torch.zeros(nb, hkv, bs, d, dtype=BF16, device="cuda"); vc = torch.zeros_like(kc)
    q2, kc2, vc2 = qkv.cpu().clone(), kc.cpu().clone(), vc.cpu().clone()
    ops.rope_kv_paged(qkv, pos, slots, kc, vc, hq, hkv, d, 5e5)
    ref.rope_kv_paged(q2, pos.cpu(), slots.cpu(), kc2, vc2, hq, hkv, d, 5e5)
    ops.check_status()
    # BF16 arithmetic contract: allow one ULP from fast sin/cos differences
    _close(qkv[:, : (hq + hkv) * d], q2[:, : (hq + hkv) * d], 1e-2, 1e-2)
    _close(kc, kc2, 1e-2, 1e-2)
    assert torch.equal(vc.cpu(), vc2)


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_silu_mul(mode):
    gu = _rand((9, 2 * 1024), 18, 2.0)
    _close(ops.silu_mul(gu, mode=mode), ref.silu_mul(gu.cpu(), mode=mode), 1e-2, 1e-3)


def test_argmax_ties_lower_id():
    lg = _rand((5, 5000), 19)
    lg[0, 10] = 100.0; lg[0, 4000] = 100.0
    lg[1, :] = 0.0
    ids = ops.argmax_rows(lg)
    assert ids.cpu().tolist() == ref.argmax_rows(lg.cpu()).tolist()
    assert ids[0].item() == 10 and ids[1].item() == 0
    ops.check_status()


def _fill_cache(nb, hkv, d, seed):
    kc = _rand((nb, hkv, 64, d), seed)
    vc = _rand((nb, hkv, 64, d), seed + 1)
    return kc, vc


@pytest.mark.parametrize("batch,hq,hkv,ctxs", [(1, 4, 1, [1]), (3, 8, 2, [5, 64, 200]), (2, 32, 8, [1024, 777]),
                                                (4, 8, 1, [130, 64, 63, 65])])
def test_attn_decode(batch, hq, hkv, ctxs):
    d = 128
    max_blocks = 20
    nb = batch * max_blocks
    kc, vc = _fill_cache(nb, hkv, d, 20)
    perm = torch.randperm(nb, generator=torch.Generator().manual_seed(3)).to(torch.int32)
    bt = perm.view(batch, max_blocks).contiguous().cuda()
    ctx = torch.tensor(ctxs, dtype=torch.int32, device="cuda")
    q = _rand((batch, (hq + 2 * hkv) * d), 22)
    out = ops.attn_decode(q, kc, vc, bt, ctx, hq, hkv, d, 1 / math.sqrt(d), max_ctx=max_blocks * 64)
    ops.check_status()
    expect = ref.attention_paged(q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), torch.arange(batch, dtype=torch.int32),
                                 torch.ones(batch, dtype=torch.int32), ctx.cpu(), hq, hkv, d, 1 / math.sqrt(d))
    _close(out, expect, 2e-2, 2e-2)


def test_attn_decode_multirow_causal_and_tree():
    d, hq, hkv, batch, nq = 128, 4, 1, 2, 4
    max_blocks = 4
    kc, vc = _fill_cache(batch * max_blocks, hkv, d, 30)
    bt = torch.arange(batch * max_blocks, dtype=torch.int32).view(batch, max_blocks).cuda()
    ctx = torch.tensor([70, 133], dtype=torch.int32, device="cuda")
    q = _rand((batch * nq, hq * d), 32)
    qs = torch.arange(batch, dtype=torch.int32) * nq
    ql = torch.full((batch,), nq, dtype=torch.int32)
    out = ops.attn_decode(q, kc, vc, bt, ctx, hq, hkv, d, 0.088, nq=nq)
    expect = ref.attention_paged(q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), qs, ql, ctx.cpu(), hq, hkv, d, 0.088)
    _close(out, expect, 2e-2, 2e-2)
    # tree: row 0 root, rows 1 and 2 children of 0, row 3 child of 1
    masks = torch.tensor([[0b0001, 0b0011, 0b0101, 0b1011]] * batch, dtype=torch.int64)
    out = ops.attn_decode(q, kc, vc, bt, ctx, hq, hkv, d, 0.088, nq=nq, tree_mask=masks.cuda())
    expect = ref.attention_paged(q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), qs, ql, ctx.cpu(), hq, hkv, d, 0.088,
                                 tree_mask=masks)
    _close(out, expect, 2e-2, 2e-2)
    ops.check_status()


@pytest.mark.parametrize("qlens,pasts", [([64], [0]), ([100, 7, 129], [0, 64, 30]), ([300], [200])])
def test_attn_prefill(qlens, pasts):
    d, hq, hkv = 128, 4, 2
    batch = len(qlens)
    max_blocks = 10
    kc, vc = _fill_cache(batch * max_blocks, hkv, d, 40)
    bt = torch.arange(batch * max_blocks, dtype=torch.int32).view(batch, max_blocks).cuda()
    ql = torch.tensor(qlens, dtype=torch.int32)
    qs = torch.cumsum(ql, 0).to(torch.int32) - ql
    ctx = ql + torch.tensor(pasts, dtype=torch.int32)
    rows = int(ql.sum())
    q = _rand((rows, (hq + 2 * hkv) * d), 42)
    out = ops.attn_prefill(q, kc, vc, bt, qs.cuda(), ql.cuda(), ctx.cuda(), max(qlens), hq, hkv, d, 0.088)
    ops.check_status()
    expect = ref.attention_paged(q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), qs, ql, ctx, hq, hkv, d, 0.088)
    _close(out, expect, 2e-2, 2e-2)


def test_sampler_matches_host_reference():
    torch.manual_seed(0)
    lg = (torch.randn(4, 3000) * 3).cuda()
    for (t, k, p) in [(0.7, 50, 0.9), (1.0, 0, 0.5), (1.3, 5, 1.0)]:
        got = ops.sample_rows(lg, t, k, p, seed=1234, step=7)
        probs = [ref.sampling_probs(lg[r].cpu(), t, k, p) for r in range(4)]
        for r in range(4):
            assert probs[r][int(got[r])] > 0, "sampled id must lie in the kept set"
    # determinism
    a = ops.sample_rows(lg, 0.8, 40, 0.95, seed=5, step=1)
    b = ops.sample_rows(lg, 0.8, 40, 0.95, seed=5, step=1)
    assert torch.equal(a, b)


def test_silu_mul_interleaved_layout():
    f, m = 512, 5
    g, u = _rand((m, f), 50, 2.0), _rand((m, f), 51, 2.0)
    inter = torch.cat([g.view(m, f // 64, 1, 64), u.view(m, f // 64, 1, 64)], dim=2).reshape(m, 2 * f).contiguous()
    got = ops.silu_mul(inter, interleaved=True)
    _close(got, ref.silu_mul(torch.cat([g, u], dim=1).cpu()), 1e-2, 1e-3)


@pytest.mark.parametrize("m,n,k", [(64, 28672, 4096), (64, 4096, 14336), (3, 128256, 4096), (128, 6144, 4096),
                                   (16, 130, 64), (1, 128, 128)])
def test_gemm_skinny_streamk_shapes(m, n, k):
    """Shapes whose work units split unevenly over the persistent CTAs (partial tiles at both ends)."""
    x, w = _rand((m, k), 52), _rand((n, k), 53, 0.03)
    y = ops.linear(x, w)
    y2 = ops.linear(x, w)
    torch.cuda.synchronize()
    ops.check_status()
    assert torch.equal(y, y2), "stream-K fix-up must be deterministic"
    # reference on the GPU in FP32 (the CPU matmul of the big shapes is slow)
    expect = (x.float() @ w.float().t())
    _close(y, expect)


def test_attn_decode_many_rows_tree():
    """40 query rows x 4 heads per kv head = 10 packed row tiles, random ancestor masks."""
    d, hq, hkv, batch, nq = 128, 8, 2, 2, 40
    max_blocks = 6
    kc, vc = _fill_cache(batch * max_blocks, hkv, d, 60)
    bt = torch.arange(batch * max_blocks, dtype=torch.int32).view(batch, max_blocks).cuda()
    ctx = torch.tensor([100, 290], dtype=torch.int32, device="cuda")
    q = _rand((batch * nq, hq * d), 62)
    g = torch.Generator().manual_seed(5)
    masks = []
    for b in range(batch):
        row = []
        for r in range(nq):
            m = int(torch.randint(0, 2 ** 31, (1,), generator=g)) & ((1 << r) - 1)
            row.append(m | (1 << r))
        masks.append(row)
    masks = torch.tensor(masks, dtype=torch.int64)
    out = ops.attn_decode(q, kc, vc, bt, ctx, hq, hkv, d, 0.088, nq=nq, tree_mask=masks.cuda())
    ops.check_status()
    qs = torch.arange(batch, dtype=torch.int32) * nq
    ql = torch.full((batch,), nq, dtype=torch.int32)
    expect = ref.attention_paged(q.cpu(), kc.cpu(), vc.cpu(), bt.cpu(), qs, ql, ctx.cpu(), hq, hkv, d, 0.088,
                                 tree_mask=masks)
    _close(out, expect, 2e-2, 2e-2)


@pytest.mark.parametrize("window", [1, 37, 64, 100, 200])
def test_attn_prefill_sliding_window_is_exact(window):
    """Every row sees exactly its last ``window`` keys, also when the bound falls inside a page."""
    g = torch.Generator().manual_seed(21)
    hq, hkv, d, bs = 4, 2, 128, 64
    lens = [150, 70]
    nb = 8
    kc = (torch.randn(nb, hkv, bs, d, generator=g) * 0.5).to(torch.bfloat16)
    vc = (torch.randn(nb, hkv, bs, d, generator=g) * 0.5).to(torch.bfloat16)
    bt = torch.tensor([[0, 1, 2, 3], [4, 5, 6, 7]], dtype=torch.int32)
    rows = sum(lens)
    q = (torch.randn(rows, hq * d, generator=g) * 0.5).to(torch.bfloat16)
    q_start = torch.tensor([0, lens[0]], dtype=torch.int32)
    q_lens = torch.tensor(lens, dtype=torch.int32)
    ctx = torch.tensor([lens[0] + 40, lens[1]], dtype=torch.int32)          # the first sequence has 40 cached keys
    want = ops.attn_prefill(q, kc, vc, bt, q_start, q_lens, ctx, max(lens), hq, hkv, d, d ** -0.5, window=window)
    got = ops.attn_prefill(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), q_start.cuda(), q_lens.cuda(), ctx.cuda(), max(lens),
                           hq, hkv, d, d ** -0.5, window=window)
    ops.check_status()
    assert torch.allclose(got.float().cpu(), want.float(), rtol=3e-2, atol=3e-2)


@pytest.mark.parametrize("window", [1, 50, 64, 130])
def test_attn_decode_sliding_window(window):
    g = torch.Generator().manual_seed(22)
    hq, hkv, d, bs, batch = 8, 2, 128, 64, 3
    nb = 12
    kc = (torch.randn(nb, hkv, bs, d, generator=g) * 0.5).to(torch.bfloat16)
    vc = (torch.randn(nb, hkv, bs, d, generator=g) * 0.5).to(torch.bfloat16)
    bt = torch.arange(nb, dtype=torch.int32).reshape(batch, 4)
    ctx = torch.tensor([200, 64, 7], dtype=torch.int32)
    q = (torch.randn(batch, hq * d, generator=g) * 0.5).to(torch.bfloat16)
    want = ops.attn_decode(q, kc, vc, bt, ctx, hq, hkv, d, d ** -0.5, window=window)
    got = ops.attn_decode(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), ctx.cuda(), hq, hkv, d, d ** -0.5, window=window)
    ops.check_status()
    assert torch.allclose(got.float().cpu(), want.float(), rtol=3e-2, atol=3e-2)
    full = ops.attn_decode(q, kc, vc, bt, ctx, hq, hkv, d, d ** -0.5)
    if window < 200:
        assert not torch.allclose(want[0].float(), full[0].float(), atol=1e-3)      # the window really hides keys


def test_kv_move_rows_kernel_matches_indexing():
    """Compaction of tree-verification rows: the two-launch kernel over all layers equals gather-then-scatter by tensor
    indexing, also when source and destination positions overlap."""
    from flyingfish_b200.engine.kv_cache import PagedKVCache
    dev = torch.device("cuda", 0)
    kv = PagedKVCache(3, 2, 128, 8, 64, torch.bfloat16, dev)
    g = torch.Generator().manual_seed(9)
    for l in range(3):
        kv.k[l].copy_(torch.randn(kv.k[l].shape, generator=g).to(torch.bfloat16))
        kv.v[l].copy_(torch.randn(kv.v[l].shape, generator=g).to(torch.bfloat16))
    kv.add_sequence(0)
    kv.reserve(0, 150); kv.commit(0, 150)
    src, dst = [70, 71, 75, 130, 64], [64, 65, 66, 67, 68]          # 64 is both read and written
    want_k = [t.clone() for t in kv.k]; want_v = [t.clone() for t in kv.v]
    blocks = kv.seqs[0].blocks
    for cache in want_k + want_v:
        rows = torch.stack([cache[blocks[p // 64], :, p % 64, :].clone() for p in src])
        for i, p in enumerate(dst):
            cache[blocks[p // 64], :, p % 64, :] = rows[i]
    kv.move_rows(0, src, dst)
    torch.cuda.synchronize()
    ops.check_status(dev)
    for l in range(3):
        assert torch.equal(kv.k[l], want_k[l]) and torch.equal(kv.v[l], want_v[l])


def test_mtp_mix_and_device_accept_match_oracles():
    from flyingfish_b200.ops import spec_ops
    from flyingfish_b200.spec.accept import accept_chain
    g = torch.Generator().manual_seed(4)
    rows, h, vocab = 9, 1024, 500
    table = torch.randn(vocab, h, generator=g).to(torch.bfloat16)
    hidden = torch.randn(rows, h, generator=g).to(torch.bfloat16)
    en = (1 + 0.1 * torch.randn(h, generator=g)).to(torch.bfloat16)
    hn = (1 + 0.1 * torch.randn(h, generator=g)).to(torch.bfloat16)
    ids = torch.randint(0, vocab, (rows,), generator=g).to(torch.int32)
    want = spec_ops.mtp_mix(ids, table, hidden, en, hn, 1e-6).float()
    got = spec_ops.mtp_mix(ids.cuda(), table.cuda(), hidden.cuda(), en.cuda(), hn.cuda(), 1e-6).float().cpu()
    assert (want - got).abs().max().item() <= 2e-2
    # acceptance: every prefix length, with and without an end-of-sequence token inside the accepted prefix
    k = 4
    drafts, targets = [], []
    for n_match in range(k + 1):
        d = [10 + j for j in range(k)]
        t = [10 + j for j in range(n_match)] + [99] * (k + 1 - n_match)
        drafts.append(d); targets.append(t)
    drafts.append([10, 7, 12, 13]); targets.append([10, 7, 12, 13, 14])          # 7 is an end-of-sequence id
    dd, tt = torch.tensor(drafts, dtype=torch.int32), torch.tensor(targets, dtype=torch.int32)
    for ignore in (True, False):
        out = spec_ops.accept_chain(dd.cuda(), tt.cuda(), (7,), ignore).cpu().tolist()
        for b, row in enumerate(out):
            a = accept_chain(drafts[b], targets[b], (7,), ignore)
            assert row[0] == a.n_draft_accepted and row[1] == len(a.tokens) and bool(row[2]) == a.hit_eos
            assert row[3: 3 + row[1]] == a.tokens
