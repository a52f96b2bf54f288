"""DSA indexer (pooling, index scores, top-k, expansion) and sparse attention: oracle properties on CPU,
CUDA kernels against the oracles."""
import pytest
import torch

from flyingfish_b200.ops import dsa_ops as dsa

BF16 = torch.bfloat16


def _seqs(lens, d=256, seed=0):
    g = torch.Generator().manual_seed(seed)
    total = sum(lens)
    latent = torch.randn(total, d, generator=g).to(BF16)
    idx_key = torch.randn(total, 128, generator=g).to(BF16)
    logit = torch.randn(total, 128, generator=g).to(BF16)
    ape = torch.randn(4, 128, generator=g).to(BF16)
    seq_len = torch.tensor(lens, dtype=torch.int32)
    seq_start = (torch.cumsum(seq_len, 0) - seq_len).to(torch.int32)
    return latent, idx_key, logit, ape, seq_start, seq_len


def test_pool_topk_expand_oracle_properties():
    latent, idx_key, logit, ape, seq_start, seq_len = _seqs([37, 8])
    pooled, pool_start = dsa.pool_keys(idx_key, logit, ape, seq_start, seq_len)
    assert pooled.shape == (9 + 2, 128) and pool_start.tolist() == [0, 9]
    # a pooled key is a convex combination per channel (up to BF16 rounding)
    lo = idx_key[:4].float().min(0).values; hi = idx_key[:4].float().max(0).values
    assert ((pooled[0].float() >= lo - 0.05) & (pooled[0].float() <= hi + 0.05)).all()
    g = torch.Generator().manual_seed(9)
    q = torch.randn(2, 32, 128, generator=g).to(BF16); w = torch.rand(2, 32, generator=g).to(BF16)
    # row 0: query at position 22 of sequence 0 -> 5 complete pools; row 1: position 7 of sequence 1 -> 2 pools
    pos = torch.tensor([22, 7], dtype=torch.int32)
    n_cand = ((pos + 1) // 4).to(torch.int32)
    sel, val = dsa.index_topk(q, w, pooled, pool_start, n_cand, k=4)
    assert sorted(sel[1, :2].tolist()) == [0, 1] and sel[1, 2:].tolist() == [-1, -1]
    assert (val[0, :4][:-1] >= val[0, :4][1:]).all() and len(set(sel[0].tolist())) == 4
    idx = dsa.expand(sel, seq_start, pos)
    assert idx.shape == (2, 4 * 4 + 3)
    live0 = [i for i in idx[0].tolist() if i >= 0]
    assert len(live0) == 16 + 3 and set(live0[-3:]) == {20, 21, 22}                 # tail tokens 20..22
    live1 = [i for i in idx[1].tolist() if i >= 0]
    assert sorted(live1) == list(range(37, 45))                                       # both pools of sequence 1, no tail


def test_sparse_attention_oracle_ignores_unselected_rows():
    latent, *_ = _seqs([40], d=128, seed=2)
    g = torch.Generator().manual_seed(3)
    q = torch.randn(1, 4, 128, generator=g).to(BF16); sink = torch.zeros(4)
    idx = torch.tensor([[3, 7, -1, 11]], dtype=torch.int32)
    out = dsa.sparse_attention(q, latent, idx, sink)
    latent2 = latent.clone(); latent2[20:] += 5.0                                     # not selected -> no effect
    assert torch.equal(out, dsa.sparse_attention(q, latent2, idx, sink))
    none = dsa.sparse_attention(q, latent, torch.full((1, 4), -1, dtype=torch.int32), sink)
    assert none.abs().max() == 0                                                      # only the sink: zero output


@pytest.mark.gpu
def test_dsa_cuda_matches_oracles():
    from flyingfish_b200 import ops
    lens = [1029, 4, 263, 2600]
    latent, idx_key, logit, ape, seq_start, seq_len = _seqs(lens, d=512, seed=5)
    pooled, pool_start = dsa.pool_keys(idx_key, logit, ape, seq_start, seq_len)
    cu = lambda t: t.cuda()
    pooled_g, pool_start_g = dsa.pool_keys(cu(idx_key), cu(logit), cu(ape), cu(seq_start), cu(seq_len))
    assert torch.equal(pool_start_g.cpu(), pool_start)
    assert (pooled_g.float().cpu() - pooled.float()).abs().max() <= 2e-2
    g = torch.Generator().manual_seed(6)
    rows_seq = [0, 0, 1, 2, 3, 3]
    pos = torch.tensor([1028, 500, 3, 262, 2599, 2100], dtype=torch.int32)
    q = torch.randn(6, 32, 128, generator=g).to(BF16); w = torch.rand(6, 32, generator=g).to(BF16)
    pool_base = pool_start[rows_seq].contiguous(); seq_base = seq_start[rows_seq].contiguous()
    n_cand = ((pos + 1) // 4).to(torch.int32)
    # score with the CUDA-pooled keys on both sides so the ranking sees identical inputs
    sel, val = dsa.index_topk(q, w, pooled_g.cpu(), pool_base, n_cand, k=512)
    sel_g, val_g = dsa.index_topk(cu(q), cu(w), pooled_g, cu(pool_base), cu(n_cand), k=512)
    ops.check_status()
    assert (val_g.cpu()[val > -1e30] - val[val > -1e30]).abs().max() <= 1e-3
    for r in range(6):
        a, b = sel[r].tolist(), sel_g[r].cpu().tolist()
        assert sum(i >= 0 for i in a) == sum(i >= 0 for i in b)
        # same set except where scores tie within FP32 summation-order noise
        assert len(set(a) ^ set(b)) <= 4, (r, len(set(a) ^ set(b)))
    idx_g = dsa.expand(sel_g, cu(seq_base), cu(pos))
    assert torch.equal(idx_g.cpu(), dsa.expand(sel_g.cpu(), seq_base, pos))
    qa = torch.randn(6, 24, 512, generator=g).to(BF16); sink = torch.randn(24, generator=g)
    want = dsa.sparse_attention(qa, latent, idx_g.cpu(), sink)
    got = dsa.sparse_attention(cu(qa), cu(latent), idx_g, cu(sink))
    ops.check_status()
    err = (got.float().cpu() - want.float()).abs().max().item()
    assert err <= 2e-2 + 2e-2 * want.float().abs().max().item(), err


@pytest.mark.gpu
def test_dsa_topk_ties_prefer_lower_id():
    from flyingfish_b200 import ops
    # identical pooled keys -> identical scores: the k lowest ids win, in ascending order
    pooled = torch.ones(40, 128, dtype=BF16, device="cuda")
    q = torch.ones(1, 32, 128, dtype=BF16, device="cuda"); w = torch.ones(1, 32, dtype=BF16, device="cuda")
    sel, val = dsa.index_topk(q, w, pooled, torch.zeros(1, dtype=torch.int32, device="cuda"),
                              torch.tensor([40], dtype=torch.int32, device="cuda"), k=16)
    ops.check_status()
    assert sel[0].cpu().tolist() == list(range(16))
