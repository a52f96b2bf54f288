"""Calibrated kernel choices: the decode-GEMM decomposition table and the split-KV wave target of decode attention.
Every decomposition a calibration run may install must compute the same product; the table is keyed without the row
count, so a row's bits cannot depend on the batch it is computed in."""
import ctypes

import pytest
import torch

from flyingfish_b200.config import named_shape
from flyingfish_b200.planner import calibrate as cal


def test_decode_shapes_and_candidates():
    s = named_shape("llama3-8b-shape")
    shapes = {n: (a, b, e) for n, a, b, e in cal.decode_linear_shapes(s)}
    assert shapes == {"qkv": (6144, 4096, 2), "o": (4096, 4096, 0), "gate_up": (28672, 4096, 1), "down": (4096, 14336, 0)}
    assert cal.decode_linear_shapes(s, tp=8)[3][1:] == (4096, 14336 // 8, 0)
    assert (1, 128) in cal.linear_candidates(0) and all(r == 128 for _, r in cal.linear_candidates(1))
    assert cal.apply_kernel_choices(None) == 0 and cal.apply_kernel_choices({}) == 0


@pytest.mark.gpu
def test_every_installable_decomposition_is_correct_and_batch_invariant():
    from flyingfish_b200 import ops
    from flyingfish_b200.ops.lib import kernels
    lib = kernels()
    g = torch.Generator().manual_seed(0)
    n, k = 4096, 4096
    x = torch.randn(64, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).cuda()
    want = (x.float() @ w.float().t())
    seen = 0
    try:
        for s_, r_ in cal.linear_candidates(0):
            lib.ff_gemm_skinny_set_choice(n, k, 0, s_, r_)
            cfg = (ctypes.c_int * 5)()
            lib.ff_gemm_skinny_config(64, n, k, 0, cfg)
            if (cfg[0], cfg[1]) != (s_, r_):
                continue
            seen += 1
            y64 = ops.linear(x, w)
            assert (y64.float() - want).abs().max() <= 2e-2 * want.abs().max(), (s_, r_)
            # the same rows computed in a batch of 5 give the same bits: the K split is fixed per (N, K)
            assert torch.equal(ops.linear(x[:5].contiguous(), w), y64[:5]), (s_, r_)
        assert seen >= 4
    finally:
        lib.ff_gemm_skinny_set_choice(n, k, 0, 0, 0)
    ops.check_status()


@pytest.mark.gpu
def test_measure_and_apply_choices_on_a_small_shape():
    from flyingfish_b200 import ops
    from flyingfish_b200.ops.lib import kernels
    spec = named_shape("tiny-llama")
    res = cal.measure_linear_choices(spec, m=16, iters=4)
    assert set(res) == {"qkv", "o", "gate_up", "down"} and all(v["us"] <= v["default_us"] for v in res.values())
    plan = cal.measure_attention_plan(spec, cases=((4, 600),), iters=3)
    assert plan["waves"] in (1, 2, 4, 8)
    assert cal.apply_kernel_choices({"linear_choices": res, "attention_plan": plan}) >= 0
    # leave the library on its defaults for the tests that follow
    for v in res.values():
        for e in (0, 1, 2):
            kernels().ff_gemm_skinny_set_choice(v["n"], v["k"], e, 0, 0)
    kernels().ff_attn_decode_set_waves(4)
    ops.check_status()


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(128, 8192, 1024), (128, 8192, 3584), (96, 8192, 3584), (128, 6144, 4096)])
def test_many_tokens_on_a_wide_cluster_tile(m, n, k):
    """A cluster split chosen for 64 tokens with 256-row tiles leaves too little shared memory for 128 tokens: the
    tile is narrowed for that launch, the K split (and with it every output bit) stays the same."""
    from flyingfish_b200 import ops
    g = torch.Generator().manual_seed(1)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).cuda()
    y = ops.linear(x, w)
    want = x.float() @ w.float().t()
    assert (y.float() - want).abs().max() <= 2e-2 * want.abs().max()
    assert torch.equal(ops.linear(x[:7].contiguous(), w), y[:7])
    assert torch.equal(ops.linear(x[:64].contiguous(), w), y[:64])
    ops.check_status()
