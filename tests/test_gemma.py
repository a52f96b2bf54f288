"""Gemma-layout decoder: sliding-window local layers stay consistent between prefill, chunked prefill and decode."""
import pytest
import torch

from flyingfish_b200.api import Model, generate_plain
from flyingfish_b200.config import Settings


def _load(device="cpu"):
    return Model.load("tiny-gemma", Settings(capacity=256, max_batch=4, graph=False), device=device, seed=0)


def _check(m):
    net = m.engine.model
    assert [net.is_global(i) for i in range(6)] == [False] * 5 + [True]
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, 2000, (120,), generator=g).tolist()          # longer than the window of 48
    out = generate_plain(m, prompt, 6, ignore_eos=True, graph=False).ids
    for k in (1, 4):
        m.reset()
        assert m.prefill(prompt + out[:k]) == out[k], k                   # decode == whole-prompt prefill
    m.reset()
    m.engine.settings.chunk = 32
    assert m.prefill(prompt + out[:2]) == out[2]                          # chunked prefill across the window edge
    m.engine.settings.chunk = 0
    return out


def test_gemma_cpu_window_consistency():
    m = _load()
    _check(m)
    # the window matters: a model with a huge window gives different logits on a long prompt
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, 2000, (120,), generator=g).tolist()
    from flyingfish_b200.models.encoder import run_whole
    a = run_whole(m, [prompt], "hidden")[0][-1].float()
    m.engine.model.window = 10 ** 6
    b = run_whole(m, [prompt], "hidden")[0][-1].float()
    assert (a - b).abs().max() > 1e-4


@pytest.mark.gpu
def test_gemma_gpu_window_consistency():
    from flyingfish_b200 import ops
    _check(_load("cuda"))
    ops.check_status()


@pytest.mark.gpu
def test_gemma_gpu_matches_cpu_oracle():
    from _oracle import assert_hidden_close
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, 2000, (120,), generator=g).tolist()
    # the unnormalised residual stream of the sandwich-norm layout grows to ~15 by the last layer, where one BF16 step
    # is 0.06-0.12 and every layer roughly doubles the accumulated difference: measured 0.09 of scale, cosine 0.9986
    assert_hidden_close(_load(), _load("cuda"), [prompt, [4, 5, 6, 7]], rel=0.15)
