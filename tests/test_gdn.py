"""Gated DeltaNet: the recurrence equals its closed matrix form, history carries across calls, CUDA == oracle."""
import pytest
import torch

from flyingfish_b200.ops import gdn_ops as gdn

BF16 = torch.bfloat16


def _rows(rows, heads, kheads, seed=0):
    g = torch.Generator().manual_seed(seed)
    ch = (2 * kheads + heads) * 128
    x = torch.randn(rows, ch, generator=g).to(BF16)
    w = (torch.randn(ch, 4, generator=g) * 0.5).to(BF16)
    beta = torch.rand(rows, heads, generator=g); gate = -torch.rand(rows, heads, generator=g) * 0.2
    return x, w, beta, gate


def test_conv_history_and_recurrence_matrix_form():
    x, w, beta, gate = _rows(6, 2, 1)
    hist = torch.zeros(x.shape[1], 3)
    whole = gdn.conv(x, w, hist.clone())
    h2 = hist.clone()
    parts = torch.cat([gdn.conv(x[:2], w, h2), gdn.conv(x[2:], w, h2)])
    assert torch.equal(whole, parts)                                   # the history makes split calls identical
    q, k, v = gdn.prep(whole, 2, 1)
    assert torch.allclose((k * k).sum(-1), torch.ones(6, 2), atol=1e-3)
    S = torch.zeros(1, 2, 128, 128)
    out = gdn.recurrent(q, k, v, beta, gate, S, torch.tensor([0, 6], dtype=torch.int32))
    # closed form: S_t = exp(g)(I - beta k k^T) S_{t-1} + beta k v^T
    Sm = torch.zeros(2, 128, 128)
    for r in range(6):
        for h in range(2):
            kk = k[r, h][:, None]
            Sm[h] = torch.exp(gate[r, h]) * (torch.eye(128) - beta[r, h] * kk @ kk.t()) @ Sm[h] + beta[r, h] * kk @ v[r, h][None, :]
    assert torch.allclose(S[0], Sm, atol=1e-4)
    assert torch.allclose(out[5].float(), torch.einsum("hk,hkv->hv", q[5], Sm), atol=2e-2)


@pytest.mark.gpu
def test_gdn_cuda_matches_oracle():
    heads, kheads = 8, 2
    x, w, beta, gate = _rows(21, heads, kheads, seed=1)
    hist = torch.randn(x.shape[1], 3, generator=torch.Generator().manual_seed(2))
    hc, hg = hist.clone(), hist.clone().cuda()
    want = gdn.conv(x, w, hc); got = gdn.conv(x.cuda(), w.cuda(), hg)
    assert (got.float().cpu() - want.float()).abs().max() <= 3e-2 and torch.allclose(hg.cpu(), hc)
    q, k, v = gdn.prep(want, heads, kheads); qg, kg, vg = gdn.prep(want.cuda(), heads, kheads)
    for a, b in ((qg, q), (kg, k), (vg, v)):
        assert (a.cpu() - b).abs().max() <= 1e-5
    rs = torch.tensor([0, 9, 10, 21], dtype=torch.int32)
    S = torch.randn(3, heads, 128, 128, generator=torch.Generator().manual_seed(3)) * 0.05
    Sg = S.clone().cuda()
    out = gdn.recurrent(q, k, v, beta, gate, S, rs)
    outg = gdn.recurrent(qg, kg, vg, beta.cuda(), gate.cuda(), Sg, rs.cuda())
    assert (Sg.cpu() - S).abs().max() <= 1e-4
    assert (outg.float().cpu() - out.float()).abs().max() <= 2e-2
    # decode step after the prefill: one more row per sequence continues from the stored state
    x2, _, b2, g2 = _rows(3, heads, kheads, seed=4)
    c2 = gdn.conv(x2[:1].cuda(), w.cuda(), hg)
    assert c2.shape == (1, x.shape[1])


@pytest.mark.gpu
@pytest.mark.parametrize("lens", [[64], [200, 37, 1], [130, 64, 65]])
def test_chunked_prefill_form_matches_the_recurrence(lens):
    """The chunked (WY, tensor-core) form against the token-by-token oracle: outputs and final state agree to BF16
    accuracy, for full chunks, ragged tails and a non-zero incoming state."""
    from flyingfish_b200 import ops
    from flyingfish_b200.ops import gdn_ops
    g_ = torch.Generator().manual_seed(7)
    heads, rows = 3, sum(lens)
    q = torch.randn(rows, heads, 128, generator=g_); k = torch.randn(rows, heads, 128, generator=g_)
    q = q / q.norm(dim=-1, keepdim=True) * 128 ** -0.5
    k = k / k.norm(dim=-1, keepdim=True)
    v = torch.randn(rows, heads, 128, generator=g_)
    beta = torch.sigmoid(torch.randn(rows, heads, generator=g_))
    dec = -torch.rand(rows, heads, generator=g_) * 0.3
    nslots = len(lens) + 2
    state0 = torch.randn(nslots, heads, 128, 128, generator=g_) * 0.1
    rs = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    slots = torch.tensor(list(range(nslots - 1, nslots - 1 - len(lens), -1)), dtype=torch.int32)
    s_ref = state0.clone()
    want = gdn_ops.recurrent_slots(q, k, v, beta, dec, s_ref, rs, slots).float()
    s_gpu = state0.clone().cuda()
    got = gdn_ops.chunked_slots(q.cuda(), k.cuda(), v.cuda(), beta.cuda(), dec.cuda(), s_gpu, rs.cuda(), slots.cuda()).float().cpu()
    ops.check_status()
    scale = want.abs().max().item()
    assert (got - want).abs().max().item() <= 0.03 * scale, ((got - want).abs().max().item(), scale)
    sd = (s_gpu.cpu() - s_ref).abs().max().item()
    assert sd <= 0.03 * s_ref.abs().max().item(), sd
    assert torch.equal(s_gpu.cpu()[0], state0[0])                     # untouched slot
