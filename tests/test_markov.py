"""Markov head: oracle on CPU, CUDA against the oracle, batch invariance."""
import pytest
import torch

from flyingfish_b200.ops import markov_ops as mk

BF16 = torch.bfloat16


def _inputs(v, rows, p, seed=0):
    g = torch.Generator().manual_seed(seed)
    w1 = (torch.randn(v, 256, generator=g) * 0.2).to(BF16); w2 = (torch.randn(v, 256, generator=g) * 0.2).to(BF16)
    base = (torch.randn(rows, v, generator=g) * 2).to(BF16)
    tok = torch.randint(0, v, (p,), generator=g).to(torch.int32); row = torch.randint(0, rows, (p,), generator=g).to(torch.int32)
    return w1, w2, base, tok, row


def test_markov_oracle_consistency():
    w1, w2, base, tok, row = _inputs(600, 3, 4)
    top4, logp, lse = mk.markov_top4(w1, w2, base, tok, row)
    assert (logp[:, :-1] >= logp[:, 1:]).all() and (logp <= 0).all()
    assert torch.isfinite(lse).all() and top4.min() >= 0 and top4.max() < 600


@pytest.mark.gpu
def test_markov_cuda_matches_oracle_and_is_batch_invariant():
    w1, w2, base, tok, row = _inputs(9000, 5, 6, seed=2)
    w2[3000] = w2[7]                                                # same bias ...
    base[1, 7] = base[1, 3000] = 30.0                               # ... same logit: a tie at the top, lower id first
    row[0] = 1
    cu = lambda t: t.cuda()
    top4, logp, lse = mk.markov_top4(cu(w1), cu(w2), cu(base), cu(tok), cu(row))
    # oracle on the GPU-produced bias rounding: recompute with the same GEMM output is implied by tolerance on values
    t_ref, lp_ref, lse_ref = mk.markov_top4(w1, w2, base, tok, row)
    assert (lse.cpu() - lse_ref).abs().max() <= 5e-2
    agree = (top4.cpu() == t_ref).float().mean().item()
    assert agree >= 0.8                                              # BF16 ties between near-equal scores may reorder
    assert top4[0, 0].item() == 7 and top4[0, 1].item() == 3000 and float(logp[0, 0]) == float(logp[0, 1])
    one = mk.markov_top4(cu(w1), cu(w2), cu(base), cu(tok[2:3]), cu(row[2:3]))
    assert torch.equal(one[0][0], top4[2]) and torch.equal(one[1][0], logp[2]) and torch.equal(one[2][0], lse[2])
