"""Hyper-connection mixing: oracle properties (Sinkhorn makes the combination matrix nearly doubly
stochastic) and CUDA kernels against the oracle."""
import pytest
import torch

from flyingfish_b200.ops import mhc_ops as mhc

BF16 = torch.bfloat16


def _inputs(rows, mult, hidden, seed=0):
    g = torch.Generator().manual_seed(seed)
    stream = torch.randn(rows, mult, hidden, generator=g).to(BF16)
    fn = (torch.randn((2 + mult) * mult, mult * hidden, generator=g) * 0.05).to(BF16)
    base = torch.randn((2 + mult) * mult, generator=g) * 0.3
    scale = torch.tensor([0.7, 1.1, 0.9])
    sub = torch.randn(rows, hidden, generator=g).to(BF16)
    return stream, fn, base, scale, sub


def test_mixes_oracle_sinkhorn_and_ranges():
    stream, fn, base, scale, sub = _inputs(5, 4, 256)
    pre, post, comb = mhc.mixes(stream, fn, base, scale, iters=20, eps=1e-6, norm_eps=1e-6)
    assert (pre > 0).all() and (pre < 1.001).all() and (post > 0).all() and (post < 2).all()
    assert torch.allclose(comb.sum(1), torch.ones(5, 4), atol=1e-3) and torch.allclose(comb.sum(2), torch.ones(5, 4), atol=1e-2)
    y = mhc.collapse(stream, pre)
    assert y.shape == (5, 256)
    a = mhc.update(sub, stream, post, comb, 0, 0); b = mhc.update(sub, stream, post, comb.transpose(1, 2).contiguous(), 0, 1)
    assert torch.equal(a, b)                                   # orientation 1 applies the transposed matrix


@pytest.mark.gpu
@pytest.mark.parametrize("rows,mult,hidden", [(7, 4, 7168), (64, 2, 4096), (3, 8, 512)])
def test_mhc_cuda_matches_oracle(rows, mult, hidden):
    stream, fn, base, scale, sub = _inputs(rows, mult, hidden, seed=1)
    pre, post, comb = mhc.mixes(stream, fn, base, scale, 4, 1e-6, 1e-6)
    cu = lambda t: t.cuda()
    pre_g, post_g, comb_g = mhc.mixes(cu(stream), cu(fn), cu(base), cu(scale), 4, 1e-6, 1e-6)
    for a, b in ((pre_g, pre), (post_g, post), (comb_g, comb)):
        assert (a.cpu() - b).abs().max().item() <= 2e-3
    y = mhc.collapse(cu(stream), pre_g)
    assert (y.float().cpu() - mhc.collapse(stream, pre_g.cpu()).float()).abs().max().item() <= 4e-2
    for rounding in (0, 1):
        for orientation in (0, 1):
            got = mhc.update(cu(sub), cu(stream), post_g, comb_g, rounding, orientation)
            want = mhc.update(sub, stream, post_g.cpu(), comb_g.cpu(), rounding, orientation)
            assert (got.float().cpu() - want.float()).abs().max().item() <= 6e-2, (rounding, orientation)
