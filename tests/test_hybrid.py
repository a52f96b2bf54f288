"""Hybrid gated-delta-net / attention decoder: the recurrent state carried through chunked prefill and decode
gives the same result as one whole-prompt pass; GPU against CPU."""
import pytest
import torch

from flyingfish_b200.api import Model, generate_plain
from flyingfish_b200.config import Settings


def _load(device="cpu", **kw):
    return Model.load("tiny-hybrid", Settings(capacity=256, max_batch=4, graph=False, **kw), device=device, seed=0)


def test_layers_alternate_and_state_is_sized():
    m = _load()
    net = m.engine.model
    assert sorted(net.gdn_layers) == [0, 1, 2]
    assert net.state_bytes_per_sequence() == 3 * 4 * ((2 * 2 + 4) * 128 * 3 + 4 * 128 * 128)


def test_decode_equals_whole_prompt_prefill():
    m = _load()
    prompt = [5, 9, 100, 33, 7, 8, 250, 11, 12]
    out = generate_plain(m, prompt, 6, ignore_eos=True, graph=False).ids
    # feeding prompt + the first k generated tokens as a fresh prompt must continue with token k+1
    for k in (1, 3, 5):
        m.reset()
        assert m.prefill(prompt + out[:k]) == out[k], k
    # chunked prefill carries conv history and state across chunks
    m.reset()
    m.engine.settings.chunk = 4
    assert m.prefill(prompt + out[:3]) == out[3]


def test_batched_sequences_keep_their_own_state():
    m = _load()
    a, b = [5, 9, 100, 33], [7, 7, 8, 250, 11, 12, 90]
    together = m.generate_batch([a, b], 5)
    m.reset()
    alone = [generate_plain(m, a, 5, ignore_eos=True, graph=False).ids]
    m.reset()
    alone.append(generate_plain(m, b, 5, ignore_eos=True, graph=False).ids)
    assert together == alone
    # slots return to the pool
    m.reset()
    assert len(m.engine.state_slots) == m.engine.model.state_slot_count - 1


@pytest.mark.gpu
def test_hybrid_gpu_runs_and_is_self_consistent():
    m = _load("cuda")
    prompt = [5, 9, 100, 33, 7, 8, 250, 11, 12]
    out = generate_plain(m, prompt, 6, ignore_eos=True, graph=False).ids
    m.reset()
    assert m.prefill(prompt + out[:3]) == out[3]
    from flyingfish_b200 import ops
    ops.check_status()
    m.reset()
    a, b = [5, 9, 100, 33], [7, 7, 8, 250, 11, 12, 90]
    together = m.generate_batch([a, b], 5)
    m.reset()
    assert together[0] == generate_plain(m, a, 5, ignore_eos=True, graph=False).ids


@pytest.mark.gpu
def test_hybrid_gpu_matches_cpu_oracle():
    from _oracle import assert_hidden_close
    prompts = [[5, 9, 100, 33, 7, 8, 250, 11, 12, 90, 14], [3, 4, 5]]
    assert_hidden_close(_load("cpu"), _load("cuda"), prompts)


@pytest.mark.gpu
def test_hybrid_decode_replays_from_cuda_graphs():
    """State slots and row ranges are views of the packed step metadata, so the decode step of the hybrid model is
    captured per bucket; graph replays give the tokens of eager launches."""
    from flyingfish_b200.api import Model
    from flyingfish_b200.config import Settings
    g = torch.Generator().manual_seed(12)
    prompts = [torch.randint(0, 2048, (n,), generator=g).tolist() for n in (33, 7, 18)]
    eager = Model.load("tiny-hybrid", Settings(capacity=256, max_batch=4, graph=False), device="cuda", seed=0)
    graph = Model.load("tiny-hybrid", Settings(capacity=256, max_batch=4, graph=True), device="cuda", seed=0)
    assert graph.engine.use_graph
    want, got = eager.generate_batch(prompts, 12), graph.generate_batch(prompts, 12)
    assert got == want and graph.engine.stats["graph_replays"] > 0
    # a second batch reuses the capture with other slots
    again = graph.generate_batch(prompts[::-1], 12)
    assert again == want[::-1]
